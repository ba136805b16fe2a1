"""Sovozen without a GPU: its configuration, its place in the registry, its weight plan, a random model folder, and
the plain implementation checked against itself."""
import copy
import json

import numpy as np
import pytest

import plain_sovozen as plain
import sovozen_configs as sc
from burn_transformers_b200 import CheckpointError, ConfigError, config_from_folder
from burn_transformers_b200.config.registry import architecture_for
from burn_transformers_b200.config.sovozen import SovozenConfig
from burn_transformers_b200.weights import safetensors_io as st
from burn_transformers_b200.weights.loader import check, discover


def test_the_architecture_key_picks_the_model(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(sc.SMALL))
    arch, config = config_from_folder(tmp_path)
    assert arch.name == "sovozen" and isinstance(config, SovozenConfig)
    assert config.vocab == 300 and config.width == 96 and config.embedding_scale == 1.7 and config.eps == 1e-5
    assert architecture_for("Sovozen") is arch
    assert config.to_dict()["layers"] == sc.SMALL["layers"]


def broken(change):
    data = copy.deepcopy(sc.SMALL)
    change(data)
    return data


@pytest.mark.parametrize("change, field", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d["embedding"].update(scale="x"), "embedding.scale"),
    (lambda d: d.update(layers=[]), "layers"),
    (lambda d: d["layers"][0].update(type="conv"), "layers[0].type"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "layers[0].mixer.kv_rank"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "layers[0].mixer.rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10), "layers[0].mixer.rot.dims"),
    (lambda d: d["layers"][1]["mixer"].update(decay=[0.5]), "layers[1].mixer.decay"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "layers[3].mixer.kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "layers[3].mixer.kv_from"),      # a recurrence has no latent
    (lambda d: d["layers"][5]["mixer"].update(kv_from=3), "layers[5].mixer.kv_from"),      # a reader has none of its own
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=40), "layers[3].mixer.kv_from"),     # sizes must agree
    (lambda d: d["layers"][2]["mlp"].update(kind="moe"), "layers[2].mlp.kind"),
])
def test_a_broken_configuration_names_its_field(change, field):
    with pytest.raises(ConfigError) as error:
        SovozenConfig.from_dict(broken(change))
    assert f"sovozen.{field}" in str(error.value)


def test_what_a_configuration_does_not_mention_does_not_exist():
    data = copy.deepcopy(sc.SMALL)
    data["layers"][2].pop("mlp")
    data.pop("logit_scale")
    data["embedding"].pop("scale")
    data["layers"][2]["mixer"].update(rot_dim=0)
    data["layers"][2]["mixer"].pop("rot")
    data["layers"][5]["mixer"].update(rot_dim=0)
    data["layers"][5]["mixer"].pop("rot")
    config = SovozenConfig.from_dict(data)
    assert config.logit_scale == 1.0 and config.embedding_scale == 1.0
    plan = architecture_for("Sovozen").build(config)
    assert plan.blocks[2].feed_forward is None and plan.blocks[2].mixer.rot_dim == 0
    assert "l2.norm2" not in plan.weights.stored() and plan.cache_needs()[2].kv.head_dim == 40


def test_the_plan_follows_the_layer_list():
    arch = architecture_for("Sovozen")
    plan = arch.build(SovozenConfig.from_dict(sc.SMALL))
    assert [(c.block, c.cache) for c in plan.schedule] == [(0, None), (1, None), (2, None), (3, 0), (4, None), (5, 2)]
    needs = plan.cache_needs()
    assert needs[0].kv.head_dim == 48 + 8 and needs[0].kv.n_kv_heads == 1 and not needs[0].kv.has_values
    assert needs[2].kv.head_dim == 40 + 12
    assert needs[3].kv is None and needs[5].kv is None and not needs[3].states
    assert needs[1].states[0].shape == (3, 16, 24) and needs[4].states[0].shape == (1, 40, 8)
    stored = plan.weights.stored()
    assert stored["l0.mix.q"].shape == (4 * (24 + 8), 96) and stored["l0.mix.dkv"].shape == (48 + 8, 96)
    assert stored["l0.mix.uk"].shape == (4 * 24, 48) and stored["l0.mix.uv"].shape == (4 * 40, 48)
    assert "l3.mix.dkv" not in stored and "l3.mix.dkv.norm" not in stored and stored["l3.mix.sink"].shape == (6,)
    assert stored["l1.mix.v"].shape == (3 * 24, 96) and stored["l1.mix.norm"].shape == (3 * 24,)
    assert "l4.norm2" not in stored and "l4.mlp.gate" not in stored and stored["l5.mlp.down"].shape == (96, 96)
    assert stored["head"].shape == (300, 96) and stored["final.norm"].shape == (96,)


def test_a_random_folder_loads_and_a_missing_tensor_is_named(tmp_path):
    folder = sc.make_folder(tmp_path / "m", sc.SMALL, seed=5)
    arch, config = config_from_folder(folder)
    plan = arch.build(config)
    check(plan.weights, discover(folder))
    header = st.read_header(folder / "model.safetensors")
    assert tuple(header["l0.mix.sink"].shape) == (4,)
    kept = {name: st.read_tensor(entry) for name, entry in header.items() if name != "l2.mix.uk"}
    st.write_file(folder / "model.safetensors", kept)
    with pytest.raises(CheckpointError) as error:
        check(plan.weights, discover(folder))
    assert error.value.missing == ["l2.mix.uk"]


# ---- the plain implementation against itself ---------------------------------------------------------------------

def test_plain_rotation_keeps_lengths_and_relative_angles():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 3, 10))
    turned = plain.rotate_interleaved(x, np.arange(6), 6, 100.0)
    assert np.allclose(np.linalg.norm(turned, axis=-1), np.linalg.norm(x, axis=-1))
    assert np.array_equal(turned[..., 6:], x[..., 6:]) and np.allclose(turned[0], x[0])
    # the product of a turned query and a turned key depends on the distance of their positions only
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    at = lambda v, p: plain.rotate_interleaved(v, [p], 6, 100.0)[0, 0]
    assert np.isclose(at(q, 9) @ at(k, 4), at(q, 105) @ at(k, 100))


def test_plain_lightning_equals_the_sum_it_unrolls_to():
    rng = np.random.default_rng(1)
    T, width, m = 9, 12, {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.5, 0.9]}
    w = {"q": rng.standard_normal((6, width)), "k": rng.standard_normal((6, width)), "v": rng.standard_normal((8, width)),
         "g": rng.standard_normal((8, width)), "o": rng.standard_normal((width, 8)), "norm": rng.standard_normal(8)}
    h = rng.standard_normal((T, width))
    got = plain.lightning(h, m, w, "", 1e-5)
    q = plain.silu(h @ w["q"].T).reshape(T, 2, 3)
    k = plain.silu(h @ w["k"].T).reshape(T, 2, 3)
    v = plain.silu(h @ w["v"].T).reshape(T, 2, 4)
    out = np.zeros((T, 2, 4))
    for head, lam in enumerate(m["decay"]):
        for t in range(T):
            for s in range(t + 1):
                out[t, head] += lam ** (t - s) * (q[t, head] @ k[s, head]) * v[s, head]
    want = (plain.rms_norm(out.reshape(T, 8), w["norm"], 1e-5) * plain.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert np.allclose(got, want)


def test_plain_sink_takes_weight_without_adding_a_value():
    scores = np.array([[0.0, -np.inf], [1.0, 2.0]])
    values = np.array([[1.0], [3.0]])
    none = plain.sink_softmax_mix(scores, -np.inf, values)
    assert np.allclose(none[0], 1.0)
    some = plain.sink_softmax_mix(scores, 0.0, values)
    assert np.allclose(some[0], 0.5)               # one key of score 0 and a sink of 0: half the weight each
    e1, e2 = np.exp(1.0), np.exp(2.0)
    assert np.allclose(some[1], (e1 * 1.0 + e2 * 3.0) / (e1 + e2 + 1.0))
