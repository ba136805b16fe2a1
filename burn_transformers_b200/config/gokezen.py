"""Gokezen's configuration: a list of layers, a run of which may be repeated.

config.json gives every size and constant:

    {"architecture": "Gokezen", "vocab": V, "width": D, "max_positions": P, "norm": {"eps": e},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size": W}}, "left_scale": a,
                           "right": {"heads", "dim", "vdim", "gate_cap"}, "right_scale": b},
                 "mlp": null | {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff", "limit"},
                         "router": {"experts", "top", "scale", "groups": {"count", "keep"}},
                         "shared": {"ff", "limit"}}}],
     "loop": {"start": i, "stop": j, "times": n}}

Sizes have no defaults: one that is missing is an error that names it.  What a configuration does not mention does not
exist: no `loop` means every layer runs once, no `mlp` no feed-forward, no `shared` no shared expert, no `groups` one
group of all experts.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import I32_MAX, ModelConfig
from .sovozen import _is_int, _is_number

LAYER_TYPES = ("parallel",)
FEED_FORWARD_KINDS = ("dense", "moe")


@dataclasses.dataclass
class GokezenConfig(ModelConfig):
    FAMILY: ClassVar[str] = "gokezen"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("Gokezen", "gokezen")

    architecture: str = dataclasses.field(default="Gokezen", metadata={"aliases": ("model_type",)})
    vocab: int = dataclasses.field(default=0, metadata={"aliases": ()})
    width: int = dataclasses.field(default=0, metadata={"aliases": ()})
    max_positions: int = dataclasses.field(default=0, metadata={"aliases": ()})
    norm: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    layers: list = dataclasses.field(default_factory=list, metadata={"aliases": ()})
    loop: dict | None = dataclasses.field(default=None, metadata={"aliases": ()})

    @property
    def model_type(self) -> str:
        return self.MODEL_TYPES[0]

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def to_dict(self) -> dict:
        data = dataclasses.asdict(self)
        if data.get("loop") is None:
            data.pop("loop", None)
        return data

    def run_order(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass it opens or None) in the order the layers run: the layers `start` .. `stop` - 1
        run `times` times in a row, each pass after the first layers and before the rest."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    # ---- checks --------------------------------------------------------------------------------------------
    def _table(self, where: str, parent: dict, name: str) -> dict:
        value = parent.get(name) if isinstance(parent, dict) else None
        if not isinstance(value, dict):
            self._fail(f"{where}.{name}" if where else name, "is missing")
        return value

    def _ints(self, where: str, table: dict, names, *, minimum: int = 1):
        for name in names:
            if name not in table:
                self._fail(f"{where}.{name}", "is missing")
            value = table[name]
            if not _is_int(value) or value < minimum or value > I32_MAX:
                self._fail(f"{where}.{name}", f"expected an integer of at least {minimum}, found {value!r}")

    def _number(self, where: str, table: dict, name: str, *, positive: bool = False):
        if name not in table:
            self._fail(f"{where}.{name}", "is missing")
        value = table[name]
        if not _is_number(value) or (positive and value <= 0):
            self._fail(f"{where}.{name}", f"expected a finite {'positive ' if positive else ''}number, found {value!r}")

    def validate(self) -> None:
        self._check_model_type(self.architecture)
        self._check_extents(("vocab", "width", "max_positions"))
        if not isinstance(self.norm, dict):
            self._fail("norm", "must be an object")
        self._number("norm", self.norm, "eps", positive=True)
        if not isinstance(self.layers, list) or not self.layers:
            self._fail("layers", "must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                self._fail(f"{where}.type", f"expected one of {list(LAYER_TYPES)}, found "
                                            f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = self._table(where, layer, "mixer")
            left = self._table(f"{where}.mixer", mixer, "left")
            self._ints(f"{where}.mixer.left", left, ("heads", "kv_heads", "dim", "vdim"))
            self._number(f"{where}.mixer.left", left, "scale")
            self._ints(f"{where}.mixer.left.mask", self._table(f"{where}.mixer.left", left, "mask"), ("size",))
            if left["heads"] % left["kv_heads"]:
                self._fail(f"{where}.mixer.left.kv_heads", f"{left['heads']} query heads cannot share {left['kv_heads']} "
                                                           f"key heads")
            right = self._table(f"{where}.mixer", mixer, "right")
            self._ints(f"{where}.mixer.right", right, ("heads", "dim", "vdim"))
            self._number(f"{where}.mixer.right", right, "gate_cap", positive=True)
            self._number(f"{where}.mixer", mixer, "left_scale")
            self._number(f"{where}.mixer", mixer, "right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in FEED_FORWARD_KINDS:
                self._fail(f"{where}.mlp.kind", f"expected one of {list(FEED_FORWARD_KINDS)}")
            if mlp["kind"] == "dense":
                self._ints(f"{where}.mlp", mlp, ("ff",))
                continue
            expert = self._table(f"{where}.mlp", mlp, "expert")
            self._ints(f"{where}.mlp.expert", expert, ("ff",))
            self._number(f"{where}.mlp.expert", expert, "limit", positive=True)
            router = self._table(f"{where}.mlp", mlp, "router")
            self._ints(f"{where}.mlp.router", router, ("experts", "top"))
            self._number(f"{where}.mlp.router", router, "scale")
            count, keep = 1, 1
            if router.get("groups") is not None:
                groups = self._table(f"{where}.mlp.router", router, "groups")
                self._ints(f"{where}.mlp.router.groups", groups, ("count", "keep"))
                count, keep = groups["count"], groups["keep"]
            if router["experts"] % count or keep > count:
                self._fail(f"{where}.mlp.router.groups", f"{router['experts']} experts are no {count} equal groups of "
                                                         f"which {keep} can be kept")
            if router["top"] > keep * (router["experts"] // count):
                self._fail(f"{where}.mlp.router.top", f"{keep} groups of {router['experts'] // count} experts cannot give "
                                                      f"{router['top']} experts")
            if mlp.get("shared") is not None:
                shared = self._table(f"{where}.mlp", mlp, "shared")
                self._ints(f"{where}.mlp.shared", shared, ("ff",))
                self._number(f"{where}.mlp.shared", shared, "limit", positive=True)
        if self.loop is not None:
            if not isinstance(self.loop, dict):
                self._fail("loop", "must be an object")
            self._ints("loop", self.loop, ("start", "stop"), minimum=0)
            self._ints("loop", self.loop, ("times",))
            if not self.loop["start"] < self.loop["stop"] <= len(self.layers):
                self._fail("loop.stop", f"layers {self.loop['start']} .. {self.loop['stop']} - 1 are no run of the "
                                        f"{len(self.layers)} layers")
