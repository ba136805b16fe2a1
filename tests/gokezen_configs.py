"""Small Gokezen configurations for the tests, and helpers to write model folders (with tensors edited where random
weights would hide a fault) and to read them for the plain implementation.  The configurations differ from one another
in every size, in the order and repetition of their layers, and in which sizes happen to be equal or one."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import burn_transformers_b200 as bt
import plain_gpt2
from burn_transformers_b200.weights.safetensors_io import write_file


def left(heads, kv_heads, dim, vdim, window, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}


def right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def layer(left_part, right_part, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mixer": {"left": left_part, "left_scale": left_scale, "right": right_part,
                                          "right_scale": right_scale}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale, *, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


# A: layers that all differ; key and value sizes differ in both directions; 3 and 1 query heads a key head; windows of 40,
# 100, 7 and 50; a recurrence with more value channels than a block holds and one with 130 key channels; experts in 3 groups of
# which 2 are kept, and experts without groups and without a shared one; a layer without a feed-forward; layers 1 and 2
# run three times, after a first layer and before a last one.
MIXED = {"architecture": "Gokezen", "vocab": 310, "width": 96, "max_positions": 700, "norm": {"eps": 1e-5},
         "layers": [layer(left(6, 2, 24, 40, 40, 0.2), right(3, 16, 24, 10.0), 0.8, 1.3, dense(160)),
                    layer(left(4, 4, 32, 16, 100, 0.18), right(2, 40, 72, 15.0), 1.5, 0.6,
                          moe(12, 3, 48, 1.2, 2.0, groups=(3, 2), shared=(80, 0.9))),
                    layer(left(2, 1, 80, 96, 7, 0.11), right(1, 130, 20, 8.0), 1.0, 1.0),
                    layer(left(3, 3, 16, 16, 50, 0.25), right(5, 8, 8, 12.0), 0.5, 2.0, moe(5, 2, 40, 2.0, 1.0))],
         "loop": {"start": 1, "stop": 3, "times": 3}}

# B: sizes that are no multiples of 8 (the kernels' element-by-element branches), an odd vocabulary, no repeated run,
# experts whose inner size is no whole 16-byte piece, one group kept of two, one expert a token.
ODD = {"architecture": "Gokezen", "vocab": 257, "width": 72, "max_positions": 300, "norm": {"eps": 1e-6},
       "layers": [layer(left(2, 2, 20, 12, 33, 0.22), right(3, 12, 10, 20.0), 1.1, 0.9, moe(6, 1, 20, 1.5, 0.7, groups=(2, 1))),
                  layer(left(5, 1, 12, 28, 300, 0.3), right(1, 36, 50, 5.0), 0.7, 1.2, dense(100))]}

# C: a width and sizes that are no whole 16-byte pieces anywhere, a single pass through a "repeated" run, a window of one
# token and one longer than any sequence, one expert.
ODDER = {"architecture": "Gokezen", "vocab": 131, "width": 52, "max_positions": 200, "norm": {"eps": 1e-5},
         "layers": [layer(left(3, 1, 6, 10, 1, 0.4), right(2, 5, 7, 3.0), 1.0, 1.0, dense(30)),
                    layer(left(1, 1, 14, 6, 1000, 0.25), right(1, 9, 3, 30.0), -0.5, 0.8, moe(1, 1, 12, 0.8, 1.0, shared=(10, 0.5)))],
         "loop": {"start": 1, "stop": 2, "times": 1}}

# D: head sizes the attention kernels take by other routes: 80 (no tensor-core prompt kernel), 112 (run as 128), 144 (beyond the
# tensor-core decode kernel), each with a window and shared key heads.
HEADS = {"architecture": "Gokezen", "vocab": 150, "width": 80, "max_positions": 300, "norm": {"eps": 1e-5},
         "layers": [layer(left(4, 2, 72, 80, 70, 0.12), right(1, 16, 16, 10.0), 1.0, 0.5),
                    layer(left(2, 1, 100, 90, 130, 0.1), right(1, 16, 16, 10.0), 1.0, 0.5, dense(64)),
                    layer(left(2, 2, 136, 20, 33, 0.09), right(1, 16, 16, 10.0), 1.0, 0.5)]}

# One mechanism at a time (a scale of zero silences the other mixer; the stream still passes the layer).
ONLY_LEFT = {"architecture": "Gokezen", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
             "layers": [layer(left(4, 2, 16, 24, 50, 0.3), right(1, 8, 8, 10.0), 1.0, 0.0)]}
ONLY_RIGHT = {"architecture": "Gokezen", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
              "layers": [layer(left(1, 1, 8, 8, 4, 0.3), right(2, 24, 40, 9.0), 0.0, 1.0)]}
ONLY_ROUTED = {"architecture": "Gokezen", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
               "layers": [layer(left(1, 1, 8, 8, 4, 0.3), right(1, 8, 8, 10.0), 0.0, 0.0,
                                moe(8, 2, 32, 1.0, 1.5, groups=(4, 2), shared=(24, 2.0)))]}
# the whole model is one repeated run
ONLY_LOOP = {"architecture": "Gokezen", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
             "layers": [layer(left(2, 1, 16, 16, 20, 0.25), right(2, 16, 16, 10.0), 1.0, 1.0, dense(96))],
             "loop": {"start": 0, "stop": 1, "times": 4}}

CONFIGS = {"mixed": MIXED, "odd": ODD, "odder": ODDER, "heads": HEADS, "only_left": ONLY_LEFT, "only_right": ONLY_RIGHT, "only_routed": ONLY_ROUTED,
           "only_loop": ONLY_LOOP}


def sharp(config: dict, factor: float = 8.0) -> dict:
    """The same model with every attention score scaled up: softmaxes close to one-hot, so that a key that is lost at a
    page's border, doubled, or seen one position outside the window moves the logits by far more than rounding does."""
    out = copy.deepcopy(config)
    for entry in out["layers"]:
        entry["mixer"]["left"]["scale"] *= factor
    return out


def long_memory(tensors: dict) -> dict:
    """Forget gates close to one and small input gates: the state still holds the first tokens after hundreds, so a
    state that is lost, zeroed or carried over to the wrong sequence shows at every later position."""
    for name in tensors:
        if name.endswith(".right.f.b"):
            tensors[name] = tensors[name] + 6.0
        if name.endswith(".right.i.b"):
            tensors[name] = tensors[name] - 1.0
    return tensors


def make_folder(path, config: dict, *, seed=3, storage="bfloat16", edit=None) -> Path:
    """A folder with random weights.  Gains and biases, which a random model has as ones and zeros, are spread out (a
    gain read at another head's place, or a bias that is left out, would not show otherwise); `edit` then changes
    tensors by name."""
    folder = bt.write_random_model(path, config, seed=seed, storage=storage)
    stored = plain_gpt2.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1000)
    tensors = {}
    for name, value in stored.items():
        value = np.array(value)
        if value.ndim == 1:
            value = value + rng.standard_normal(value.shape) * (0.25 if name.endswith(".b") else 0.2)
        tensors[name] = value
    if edit is not None:
        tensors = edit(tensors)
    as_matrix = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    write_file(folder / "model.safetensors",
               {k: torch.from_numpy(np.ascontiguousarray(v)).to(as_matrix if v.ndim == 2 else torch.float32)
                for k, v in tensors.items()})
    return folder


def load_plain(folder):
    """(configuration as a dictionary, float64 weights by checkpoint name) for plain_gokezen."""
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain_gpt2.read_safetensors(folder / "model.safetensors")


def prompts(config: dict, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab"], n).tolist() for n in lengths]
