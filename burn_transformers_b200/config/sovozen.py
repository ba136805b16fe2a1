"""Sovozen's configuration: a list of layers, each with its own mixer and sizes.

config.json gives every size and constant:

    {"architecture": "Sovozen", "vocab": V, "width": D, "embedding": {"scale": s}, "norm": {"eps": e},
     "logit_scale": t,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"dims", "base"},
                           "kv_from": j (optional)},
                 "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [one per head]}, "mlp": ...}]}

Sizes have no defaults: a size that is missing is an error that names it.  What a configuration does not mention does
not exist: a layer without an `mlp` key has no feed-forward, a missing `embedding.scale` or `logit_scale` is 1, and a
mixer without rotated channels (`rot_dim` 0) needs no `rot`.
"""
from __future__ import annotations

import dataclasses
import math
from typing import ClassVar

from ..errors import ConfigError
from .base import I32_MAX, ModelConfig

LAYER_TYPES = ("latent_attention", "lightning")
FEED_FORWARD_KINDS = ("dense",)


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _is_number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


@dataclasses.dataclass
class SovozenConfig(ModelConfig):
    FAMILY: ClassVar[str] = "sovozen"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("Sovozen", "sovozen")

    architecture: str = dataclasses.field(default="Sovozen", metadata={"aliases": ("model_type",)})
    vocab: int = dataclasses.field(default=0, metadata={"aliases": ()})
    width: int = dataclasses.field(default=0, metadata={"aliases": ()})
    embedding: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    norm: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    logit_scale: float = dataclasses.field(default=1.0, metadata={"aliases": ()})
    layers: list = dataclasses.field(default_factory=list, metadata={"aliases": ()})

    @property
    def model_type(self) -> str:
        return self.MODEL_TYPES[0]

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding.get("scale", 1.0))

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    # ---- checks --------------------------------------------------------------------------------------------
    def _ints(self, where: str, table: dict, names, *, minimum: int = 1):
        for name in names:
            if name not in table:
                self._fail(f"{where}.{name}", "is missing")
            value = table[name]
            if not _is_int(value) or value < minimum or value > I32_MAX:
                self._fail(f"{where}.{name}", f"expected an integer of at least {minimum}, found {value!r}")

    def _number(self, where: str, table: dict, name: str, *, positive: bool = False):
        if not isinstance(table, dict) or name not in table:
            self._fail(f"{where}.{name}" if where else name, "is missing")
        value = table[name]
        if not _is_number(value) or (positive and value <= 0):
            self._fail(f"{where}.{name}" if where else name,
                       f"expected a finite {'positive ' if positive else ''}number, found {value!r}")

    def validate(self) -> None:
        self._check_model_type(self.architecture)
        self._check_extents(("vocab", "width"))
        if not isinstance(self.embedding, dict):
            self._fail("embedding", "must be an object")
        if "scale" in self.embedding:
            self._number("embedding", self.embedding, "scale")
        self._number("norm", self.norm, "eps", positive=True)
        if not _is_number(self.logit_scale):
            self._fail("logit_scale", f"expected a finite number, found {self.logit_scale!r}")
        if not isinstance(self.layers, list) or not self.layers:
            self._fail("layers", "must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                self._fail(f"{where}.type", f"expected one of {list(LAYER_TYPES)}, found "
                                            f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                self._fail(f"{where}.mixer", "is missing")
            if layer["type"] == "latent_attention":
                self._check_latent(i, f"{where}.mixer", mixer)
            else:
                self._ints(f"{where}.mixer", mixer, ("heads", "dim", "vdim"))
                decay = mixer.get("decay")
                if not isinstance(decay, list) or len(decay) != mixer["heads"] or not all(_is_number(d) for d in decay):
                    self._fail(f"{where}.mixer.decay", f"expected one number per head ({mixer['heads']})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in FEED_FORWARD_KINDS:
                    self._fail(f"{where}.mlp.kind", f"expected one of {list(FEED_FORWARD_KINDS)}")
                self._ints(f"{where}.mlp", mlp, ("ff",))

    def _check_latent(self, index: int, where: str, mixer: dict) -> None:
        self._ints(where, mixer, ("heads", "dim", "vdim", "kv_rank"))
        self._ints(where, mixer, ("rot_dim",), minimum=0)
        self._number(where, mixer, "scale")
        rot = mixer.get("rot")
        if rot is None and mixer["rot_dim"] == 0:
            rot = {"dims": 0, "base": 1.0}
        if not isinstance(rot, dict):
            self._fail(f"{where}.rot", "is missing")
        self._ints(f"{where}.rot", rot, ("dims",), minimum=0)
        self._number(f"{where}.rot", rot, "base", positive=True)
        if rot["dims"] % 2 or rot["dims"] > mixer["rot_dim"]:
            self._fail(f"{where}.rot.dims", f"must be even and at most rot_dim ({mixer['rot_dim']}), found {rot['dims']}")
        source = mixer.get("kv_from")
        if source is None:
            return
        if not _is_int(source) or not 0 <= source < index:
            self._fail(f"{where}.kv_from", f"must name an earlier layer, found {source!r}")
        other = self.layers[source]
        theirs = other.get("mixer", {}) if isinstance(other, dict) else {}
        if other.get("type") != "latent_attention" or theirs.get("kv_from") is not None:
            self._fail(f"{where}.kv_from", f"layer {source} has no latent projection of its own")
        for name in ("kv_rank", "rot_dim", "rot"):
            if theirs.get(name) != mixer.get(name):
                self._fail(f"{where}.kv_from", f"layer {source} differs in `{name}`")
