"""Gokezen's configuration, plan and weights on the CPU: the registry finds the design by its `architecture` key, every
broken field is named, the run order repeats the right layers, the plan asks a checkpoint for exactly the stored tensors,
and the plain implementation agrees with itself where two of its functions overlap."""
import copy
import json

import numpy as np
import pytest

import gokezen_configs as gc
import plain_gokezen as plain
from burn_transformers_b200 import models  # noqa: F401
from burn_transformers_b200.config.gokezen import GokezenConfig
from burn_transformers_b200.config.registry import architecture_for, config_from_folder
from burn_transformers_b200.errors import CheckpointError, ConfigError
from burn_transformers_b200.models.gokezen import attention_head_size
from burn_transformers_b200.weights.loader import load_weights
from burn_transformers_b200.weights.spec import Concat, PadBlocks, Stored, resolve, stored_shapes

import torch


def test_the_registry_knows_the_design(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(gc.MIXED))
    arch, config = config_from_folder(tmp_path)
    assert arch.name == "gokezen" and isinstance(config, GokezenConfig)
    assert architecture_for("Gokezen") is arch
    assert config.to_dict()["layers"] == gc.MIXED["layers"] and config.to_dict()["loop"] == gc.MIXED["loop"]
    assert "loop" not in GokezenConfig.from_dict(gc.ODD).to_dict()


def test_run_order_repeats_the_run_and_opens_each_pass():
    config = GokezenConfig.from_dict(gc.MIXED)
    assert config.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert config.run_order() == plain.run_order(gc.MIXED)
    assert GokezenConfig.from_dict(gc.ODD).run_order() == [(0, None), (1, None)]
    assert GokezenConfig.from_dict(gc.ONLY_LOOP).run_order() == [(0, 0), (0, 1), (0, 2), (0, 3)]
    plan = architecture_for("Gokezen").build(config)
    assert [(c.block, c.opens) for c in plan.schedule] == config.run_order()
    # every call of the run owns a cache entry: keys and values of the windowed attention and the memory's state
    needs = plan.cache_needs()
    assert len(needs) == 8 and all(n.kv is not None and [s.name for s in n.states] == ["s", "n", "m"] for n in needs)


@pytest.mark.parametrize("path, value, named", [
    (("width",), 0, "width"),
    (("norm",), {}, "norm.eps"),
    (("layers", 0, "type"), "serial", "layers[0].type"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "layers[1].mixer.left.kv_heads"),
    (("layers", 0, "mixer", "left", "mask"), None, "layers[0].mixer.left.mask"),
    (("layers", 2, "mixer", "right", "gate_cap"), 0.0, "layers[2].mixer.right.gate_cap"),
    (("layers", 0, "mixer", "right_scale"), "x", "layers[0].mixer.right_scale"),
    (("layers", 0, "mlp", "kind"), "sparse", "layers[0].mlp.kind"),
    (("layers", 1, "mlp", "router", "groups", "count"), 5, "layers[1].mlp.router.groups"),
    (("layers", 1, "mlp", "router", "top"), 9, "layers[1].mlp.router.top"),
    (("layers", 1, "mlp", "shared", "limit"), -1.0, "layers[1].mlp.shared.limit"),
    (("layers", 3, "mlp", "expert"), None, "layers[3].mlp.expert"),
    (("loop", "stop"), 9, "loop.stop"),
    (("loop", "times"), 0, "loop.times"),
])
def test_a_broken_field_is_named(path, value, named):
    data = copy.deepcopy(gc.MIXED)
    at = data
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        GokezenConfig.from_dict(data)
    assert named in str(error.value)


def test_head_sizes_the_attention_runs_with():
    assert attention_head_size(16, 24) == 32 and attention_head_size(32, 16) == 32
    assert attention_head_size(24, 40) == 64 and attention_head_size(64, 64) == 64
    assert attention_head_size(80, 96) == 128 and attention_head_size(72, 8) == 80
    assert attention_head_size(130, 8) == 144


def test_padded_blocks_as_a_weight_source():
    stored = {"a": torch.arange(12.0).reshape(6, 2), "b": torch.ones(2, 2)}
    source = Concat((PadBlocks(Stored("a"), 0, 3, 4), Stored("b")), 0, (8, 2))
    assert stored_shapes(source, (10, 2)) == [("a", (6, 2)), ("b", (2, 2))]
    made = resolve(source, stored)
    assert made.shape == (10, 2) and made[3].abs().sum() == 0 and made[7].abs().sum() == 0
    assert torch.equal(made[4:7], stored["a"][3:6]) and torch.equal(made[8:], stored["b"])
    across = resolve(PadBlocks(Stored("a", transposed=True), 1, 2, 3), stored)
    assert across.shape == (2, 9) and torch.equal(across[:, 3:5], stored["a"].t()[:, 2:4]) and across[:, 5].abs().sum() == 0
    with pytest.raises(ValueError):
        stored_shapes(PadBlocks(Stored("a"), 0, 3, 4), (9, 2))


def test_the_plan_reads_exactly_the_stored_tensors(tmp_path):
    folder = gc.make_folder(tmp_path, gc.MIXED, seed=5)
    config, weights = gc.load_plain(folder)
    plan = architecture_for("Gokezen").build(GokezenConfig.from_dict(config))
    assert set(plan.weights.stored()) == set(weights)
    tensors, _ = load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    # queries, keys and values of layer 0 side by side, [in, out], heads padded from 24 / 40 channels to 64
    qkv = tensors["l0.mix.left.qkv"].numpy()
    assert qkv.shape == (96, (6 + 2 + 2) * 64)
    np.testing.assert_array_equal(qkv[:, 64:64 + 24], weights["l0.mix.left.q"][24:48].T.astype(np.float32))
    assert not qkv[:, 24:64].any() and not qkv[:, 9 * 64 + 40:].any()
    np.testing.assert_array_equal(qkv[:, 8 * 64:8 * 64 + 40], weights["l0.mix.left.v"][:40].T.astype(np.float32))
    out = tensors["l0.mix.left.out"].numpy()
    assert out.shape == (6 * 64, 96) and not out[40:64].any()
    np.testing.assert_array_equal(out[64:104], weights["l0.mix.left.o"][:, 40:80].T.astype(np.float32))
    # the memory's projections and its two gates' rows as one matrix, filled up to a multiple of 8 rows
    rows = tensors["l0.mix.right.in"].numpy()
    assert rows.shape == (2 * 48 + 2 * 72 + 8, 96)
    np.testing.assert_array_equal(rows[240:243], weights["l0.mix.right.i"].astype(np.float32))
    np.testing.assert_array_equal(rows[243:246], weights["l0.mix.right.f"].astype(np.float32))
    assert not rows[246:].any()
    experts = tensors["l1.mlp.experts.in"].numpy().reshape(12, 96, 96)
    np.testing.assert_array_equal(experts[7, 48:], weights["l1.mlp.e7.up"].astype(np.float32))
    (folder / "model.safetensors").unlink()
    del weights["l1.mlp.e3.down"]
    from burn_transformers_b200.weights.safetensors_io import write_file
    write_file(folder / "model.safetensors", {k: torch.from_numpy(v).to(torch.float32) for k, v in weights.items()})
    with pytest.raises(CheckpointError) as error:
        load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    assert "l1.mlp.e3.down" in str(error.value)


def test_the_plain_recurrence_carries_its_state():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((30, 6)), rng.standard_normal((30, 6)), rng.standard_normal((30, 4))
    a, b = plain.capped_gates(rng.standard_normal(30) * 3, rng.standard_normal(30) * 3 + 2, 6.0)
    whole, _ = plain.memory_recurrence(q, k, v, a, b)
    first, state = plain.memory_recurrence(q[:11], k[:11], v[:11], a[:11], b[:11])
    rest, _ = plain.memory_recurrence(q[11:], k[11:], v[11:], a[11:], b[11:], state)
    np.testing.assert_allclose(np.concatenate([first, rest]), whole, rtol=1e-12)
    assert np.all(a <= 6.0) and np.all(b <= 0.0)


def test_the_plain_router_keeps_to_the_best_groups():
    rng = np.random.default_rng(1)
    h, router = rng.standard_normal((50, 16)), rng.standard_normal((12, 16))
    chosen, weights = plain.route(h, router, {"experts": 12, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}})
    scores = plain.sigmoid(h @ router.T)
    for t in range(50):
        assert len({e // 4 for e in chosen[t]}) <= 2
        np.testing.assert_allclose(weights[t].sum(), 2.0, rtol=1e-12)
        assert list(scores[t, chosen[t]]) == sorted(scores[t, chosen[t]], reverse=True)
    free, _ = plain.route(h, router, {"experts": 12, "top": 3, "scale": 1.0})
    assert all(set(free[t]) == set(np.argsort(-scores[t])[:3]) for t in range(50))
