"""Two mixers in one layer, side by side."""
from __future__ import annotations

from ..cache.spec import CacheNeed
from ..errors import ShapeError
from .base import Mixer


class SideBySideMixers(Mixer):
    """Two mixers that read the same normalised rows and both add their result into the residual stream (each with the
    scale it was built with).  They share the layer's cache entry: at most one of them keeps keys and values in pages,
    and their fixed-size states must have different names."""

    def __init__(self, left: Mixer, right: Mixer):
        self.left, self.right = left, right
        a, b = left.cache_need(), right.cache_need()
        if a.kv is not None and b.kv is not None:
            raise ShapeError("mixers side by side: only one of the two may keep keys and values in pages")
        names = [s.name for s in a.states + b.states]
        if len(set(names)) != len(names):
            raise ShapeError(f"mixers side by side: their states share a name ({names})")
        self._need = CacheNeed(kv=a.kv if a.kv is not None else b.kv, states=a.states + b.states)
        # the rows are read twice, so they are real rows and no handle for a product to resolve
        self.accepts_lazy_norm = False

    def parts(self):
        return {"left": self.left, "right": self.right}

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    def cache_need(self):
        return self._need

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        self.left.forward(ctx, x, residual, entry, owns_cache)
        self.right.forward(ctx, x, residual, entry, owns_cache)
