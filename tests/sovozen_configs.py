"""Small Sovozen configurations for the tests, and helpers to write model folders and read them for the plain
implementation.  The configurations differ from one another in every size, in the order of their layers and in which
sizes happen to be equal; `sharp` variants scale the scores up so that single far keys carry the softmax."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np

import burn_transformers_b200 as bt
import plain_gpt2


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, *, rot_dims=None, base=10000.0, kv_from=None, ff=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
             "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def lightning(heads, dim, vdim, decay, *, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# A: narrow; a rotation over part of the rotated channels; a lightning layer with a feed-forward and a latent layer
# without; two latents of their own, each read by a later layer (one not the next one); heads differ between layers.
SMALL = {"architecture": "Sovozen", "vocab": 300, "width": 96, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
         "logit_scale": 0.3,
         "layers": [latent(4, 24, 8, 40, 48, 0.2, rot_dims=4, ff=160),
                    lightning(3, 16, 24, [0.9, 0.5, 1.0], ff=128),
                    latent(2, 40, 12, 16, 40, 0.15, base=500.0, ff=64),
                    latent(6, 16, 8, 8, 48, 0.3, rot_dims=4, kv_from=0),
                    lightning(1, 40, 8, [0.97]),
                    latent(3, 8, 12, 24, 40, 0.25, base=500.0, kv_from=2, ff=96)]}

# B: sizes that take the kernels' other branches: latents of 160 and 300 channels, 5 and 40 heads, recurrences with 48
# and 128 key channels and more value channels than a block holds; no scale differs from one; an odd vocabulary;
# a model that starts with a recurrence and ends with a layer without a feed-forward.
WIDE = {"architecture": "Sovozen", "vocab": 257, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "logit_scale": 1.0,
        "layers": [lightning(2, 48, 80, [0.8, 0.995], ff=192),
                   latent(5, 64, 32, 64, 160, 0.1, ff=256),
                   lightning(1, 128, 300, [0.9]),
                   latent(40, 8, 4, 8, 300, 0.3, rot_dims=2, base=100.0, ff=128),
                   latent(3, 32, 32, 48, 160, 0.12, kv_from=1)]}

# One mechanism at a time.
ONLY_LATENT = {"architecture": "Sovozen", "vocab": 120, "width": 64, "embedding": {"scale": 0.8}, "norm": {"eps": 1e-5},
               "logit_scale": 2.0, "layers": [latent(3, 16, 6, 20, 24, 0.3)]}
ONLY_LIGHTNING = {"architecture": "Sovozen", "vocab": 120, "width": 64, "embedding": {"scale": 0.8},
                  "norm": {"eps": 1e-5}, "logit_scale": 2.0, "layers": [lightning(2, 24, 20, [0.7, 0.99])]}
ONLY_SHARED = {"architecture": "Sovozen", "vocab": 120, "width": 64, "embedding": {"scale": 0.8}, "norm": {"eps": 1e-5},
               "logit_scale": 2.0, "layers": [latent(3, 16, 6, 20, 24, 0.3), latent(2, 12, 6, 28, 24, 0.2, kv_from=0)]}

CONFIGS = {"small": SMALL, "wide": WIDE, "only_latent": ONLY_LATENT, "only_lightning": ONLY_LIGHTNING,
           "only_shared": ONLY_SHARED}


def sharp(config: dict, factor: float = 8.0) -> dict:
    """The same model with every attention score scaled up: softmaxes close to one-hot, so that a key that is lost,
    doubled or seen too early moves the logits by far more than rounding does."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        if layer["type"] == "latent_attention":
            layer["mixer"]["scale"] *= factor
    return out


def make_folder(path, config: dict, *, seed=3, storage="bfloat16") -> Path:
    return bt.write_random_model(path, config, seed=seed, storage=storage)


def load_plain(folder):
    """(configuration as a dictionary, float64 weights by checkpoint name) for plain_sovozen."""
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain_gpt2.read_safetensors(folder / "model.safetensors")


def prompts(config: dict, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab"], n).tolist() for n in lengths]
