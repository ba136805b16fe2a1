"""Arrangements of norms, a mixer and a feed-forward in one layer."""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x + mixer(norm1(x)), then y + feed_forward(norm2(y)); no post-norms
    (src/models/gpt2/model.rs:218-270 of the reference).  A layer without a feed-forward (`norm2` and `feed_forward`
    None) has the first sublayer only."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None = None, feed_forward: FeedForward | None = None):
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has both a second norm and a feed-forward, or neither")
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        found = {"norm1": self.norm1, "mixer": self.mixer}
        if self.feed_forward is not None:
            found.update({"norm2": self.norm2, "feed_forward": self.feed_forward})
        return found

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx, residual, entry, owns_cache=True):
        x = self.norm1.forward(ctx, residual, ctx.dtype, lazy=self.mixer.accepts_lazy_norm)
        self.mixer.forward(ctx, x, residual, entry, owns_cache)
        if self.feed_forward is None:
            return
        x = self.norm2.forward(ctx, residual, ctx.dtype, lazy=self.feed_forward.accepts_lazy_norm)
        self.feed_forward.forward(ctx, x, residual)


class ParallelBlock(Block):
    """x + mixer(h) + feed_forward(h) with h = norm(x): one norm whose output both sublayers read, both results added
    to the stream.  A layer without a feed-forward has the mixer only."""

    def __init__(self, norm: Norm, mixer: Mixer, feed_forward: FeedForward | None = None):
        self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward

    def parts(self):
        found = {"norm": self.norm, "mixer": self.mixer}
        for name, part in getattr(self.mixer, "parts", dict)().items():
            found["mixer." + name] = part
        if self.feed_forward is not None:
            found["feed_forward"] = self.feed_forward
            for name, part in getattr(self.feed_forward, "parts", dict)().items():
                found["feed_forward." + name] = part
        return found

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx, residual, entry, owns_cache=True):
        # (both sublayers read the same rows, so the norm hands out real rows, never a handle for one product)
        x = self.norm.forward(ctx, residual, ctx.dtype, lazy=False)
        self.mixer.forward(ctx, x, residual, entry, owns_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(ctx, x, residual)
