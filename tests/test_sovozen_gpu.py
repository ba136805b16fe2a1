"""Sovozen through the engine against the plain implementation: every mechanism alone and together, whole prompts,
decoding token by token, prompts in portions, batches of unequal requests with slots and pages used again, long
decoding, sharp softmaxes, and greedy generation through the library's entry points and programs."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import engine_replay as replay
import plain_sovozen as plain
import sovozen_configs as sc
from burn_transformers_b200 import (AutoCausalLm, AutoLoadOptions, CausalGenerationRequest, Engine, GenerationConfig,
                                    StepEntry, generate_causal)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
# lengths around the borders of a page (64) and of the attention kernel's key tiles (32)
LENGTHS = {"small": [1, 2, 31, 32, 33, 63, 64, 65, 127, 129, 200], "wide": [1, 33, 64, 65, 130],
           "only_latent": [1, 5, 64, 97], "only_lightning": [1, 5, 64, 97], "only_shared": [1, 5, 64, 97]}


@pytest.fixture(scope="module", params=list(sc.CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    config = sc.CONFIGS[name]
    folder = sc.make_folder(tmp_path_factory.mktemp(name), config, seed=21)
    pcfg, pw = sc.load_plain(folder)
    seqs = sc.prompts(config, LENGTHS[name], seed=2)
    return name, folder, seqs, [plain.forward(pcfg, pw, s) for s in seqs]


def engine_for(folder, dtype, max_tokens=64 * 16, **kw):
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_whole(case, dtype):
    _, folder, seqs, ref = case
    got = replay.whole(engine_for(folder, dtype), seqs)
    err, where = replay.worst_error(got, ref)
    assert len(got) == sum(len(s) for s in seqs) and err < TOL[dtype], f"{err:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(case, dtype):
    _, folder, seqs, ref = case
    got = replay.tail_one_by_one(engine_for(folder, dtype), seqs, tail=40)
    err, where = replay.worst_error(got, ref)
    assert err < TOL[dtype], f"{err:.3e} at {where}"


def in_portions(engine, seqs, size):
    """Each request alone, `size` tokens a step."""
    got = {}
    for r, seq in enumerate(seqs):
        slot = engine.new_sequence()
        for lo in range(0, len(seq), size):
            piece = seq[lo:lo + size]
            logits = engine.step([StepEntry(slot, piece, list(range(len(piece))))]).detach().cpu().double().numpy()
            for i, row in enumerate(logits):
                got[(r, lo + i)] = row
        engine.release(slot)
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [2, 3, 31, 64, 100])
def test_prompts_in_portions(case, dtype, size):
    name, folder, seqs, ref = case
    if name != "small" and size in (3, 31):
        pytest.skip("the full set of portion sizes runs on one configuration")
    got = in_portions(engine_for(folder, dtype), seqs, size)
    err, where = replay.worst_error(got, ref)
    assert err < TOL[dtype], f"portions of {size}: {err:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_use_slots_and_pages_again(case, dtype):
    _, folder, seqs, ref = case
    n = len(seqs)
    groups = [list(range(0, n, 2)), list(range(1, n, 2)), list(range(n))[:3], list(range(n))[::-1][:3]]
    cut = [max(1, len(s) // 3) for s in seqs]
    cut[0] = 1
    need = max(sum(-(-len(seqs[r]) // 64) * 64 for r in g) for g in groups)
    engine = engine_for(folder, dtype, max_tokens=need, max_slots=max(len(g) for g in groups))
    got = replay.batches(engine, seqs, groups, cut)
    err, where = replay.worst_error(got, ref)
    assert err < TOL[dtype], f"{err:.3e} at {where}"
    assert engine.cache.slots.held == 0 and all(g.pool.held == 0 for g in engine.cache.groups)
    alone = replay.whole(engine, seqs)
    drift = max(float(np.abs(alone[k] - got[k]).max() / np.abs(ref[k[0]]).max()) for k in got)
    assert drift < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(case, dtype):
    _, folder, seqs, ref = case
    long = max(range(len(seqs)), key=lambda r: len(seqs[r]))
    got = replay.tail_one_by_one(engine_for(folder, dtype), [seqs[long]], tail=10 ** 6)
    err, where = replay.worst_error(got, [ref[long]])
    assert len(got) == len(seqs[long]) and err < TOL[dtype], f"{err:.3e} at {where}"


@pytest.mark.parametrize("plain_from", [1, 10 ** 9])
def test_both_forms_of_prompt_attention(case, plain_from, monkeypatch):
    """bfloat16 prompts of fresh sequences take the plain form (keys and values per head) from a length on and read the
    latent rows directly below it: each form alone, over all lengths, against the plain implementation; then decoding on
    top of a prompt that went through the plain form."""
    from burn_transformers_b200.parts import LatentAttention
    monkeypatch.setattr(LatentAttention, "plain_from", plain_from)
    _, folder, seqs, ref = case
    engine = engine_for(folder, "bfloat16")
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=5)):
        err, where = replay.worst_error(got, ref)
        assert err < TOL["bfloat16"], f"{err:.3e} at {where}"


def test_a_released_slot_starts_from_an_empty_state(case):
    """A sequence that takes over a slot finds neither the old recurrent state nor the old latent rows."""
    _, folder, seqs, ref = case
    engine = engine_for(folder, "float32", max_tokens=64 * 4, max_slots=1)
    for r in (len(seqs) - 1, 1, len(seqs) - 2):
        slot = engine.new_sequence()
        assert slot == 0
        got = engine.step([StepEntry(slot, seqs[r], [len(seqs[r]) - 1])]).cpu().double().numpy()[0]
        engine.release(slot)
        assert np.abs(got - ref[r][-1]).max() / np.abs(ref[r]).max() < TOL["float32"], r


@pytest.mark.parametrize("name", ["small", "wide"])
def test_sharp_softmaxes_find_single_far_keys(name, tmp_path):
    """Scores scaled up eightfold: every row's weight sits on one or two keys, often far back, so a key lost at a page's
    or a tile's border, or a reader of another layer's latent looking at the wrong rows, moves the logits visibly.
    32-bit only: rounding the scores of such a model to 8 bits moves them as much as a fault would."""
    config = sc.sharp(sc.CONFIGS[name])
    folder = sc.make_folder(tmp_path, config, seed=8)
    pcfg, pw = sc.load_plain(folder)
    seqs = sc.prompts(config, [300, 129], seed=6)
    ref = [plain.forward(pcfg, pw, s) for s in seqs]
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=70),
                replay.batches(engine, seqs, [[0, 1]], [190, 3])):
        err, where = replay.worst_error(got, ref)
        assert err < 3e-4, f"{err:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_configuration_that_leaves_out_what_it_does_not_have(tmp_path, dtype):
    """No `mlp` key, no scales, a latent layer without rotated channels and without a `rot` entry, read by a later layer."""
    config = {"architecture": "Sovozen", "vocab": 90, "width": 40, "embedding": {}, "norm": {"eps": 1e-5},
              "layers": [{"type": "latent_attention", "mixer": {"heads": 2, "dim": 12, "rot_dim": 0, "vdim": 20, "kv_rank": 16,
                                                               "scale": 0.3}},
                         sc.lightning(1, 8, 12, [0.9], ff=48),
                         {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 0, "vdim": 8, "kv_rank": 16,
                                                               "scale": 0.2, "kv_from": 0}, "mlp": None}]}
    folder = sc.make_folder(tmp_path, config, seed=3)
    pcfg, pw = sc.load_plain(folder)
    seqs = sc.prompts(config, [1, 70, 33], seed=3)
    ref = [plain.forward(pcfg, pw, s) for s in seqs]
    engine = engine_for(folder, dtype)
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=10)):
        err, where = replay.worst_error(got, ref)
        assert err < TOL[dtype], f"{err:.3e} at {where}"


def plain_greedy(pcfg, pw, prompt, n):
    seq = list(prompt)
    margins = []
    for _ in range(n):
        row = plain.forward(pcfg, pw, seq)[-1]
        order = np.argsort(row)
        margins.append(float(row[order[-1]] - row[order[-2]]))
        seq.append(int(order[-1]))
    return seq[len(prompt):], margins


@pytest.mark.parametrize("chunk", [None, 5])
def test_greedy_generation_through_the_entry_point(tmp_path, chunk):
    """Three unequal prompts as one batch through load_local and generate_causal (the scheduler, the recorded decode
    steps, the device sampler), whole prompts and prompts in portions of five: the plain implementation's tokens."""
    folder = sc.make_folder(tmp_path, sc.SMALL, seed=13)
    pcfg, pw = sc.load_plain(folder)
    prompts = sc.prompts(sc.SMALL, [3, 70, 18], seed=9)
    want = [plain_greedy(pcfg, pw, p, 12) for p in prompts]
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 4))
    out = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12),
                                                                prefill_chunk_size=chunk))
    for sequence, (tokens, margins) in zip(out.sequences, want):
        # (compared up to the first step the plain implementation itself decides by less than rounding can move)
        sure = next((i for i, m in enumerate(margins) if m < 1e-3), len(tokens))
        assert sequence.token_ids[:sure] == tokens[:sure] and sure >= 4
    bf16 = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="bfloat16", max_tokens=64 * 4))
    out16 = generate_causal(bf16.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12),
                                                               prefill_chunk_size=chunk))
    assert all(len(s.token_ids) == 12 for s in out16.sequences)
    assert sum(a == b for s, (t, _) in zip(out16.sequences, want) for a, b in zip(s.token_ids, t)) >= 18


def test_the_programs_serve_the_model(tmp_path):
    """bin/random_model writes a folder from a configuration file, bin/generate decodes from it, bin/trace_run replays a
    batch of two unequal requests on it."""
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(sc.ONLY_SHARED))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, str(ROOT / "bin" / "random_model"), str(cfg_file), str(folder), "--seed", "4"],
                          capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr
    pcfg, pw = sc.load_plain(folder)
    done = subprocess.run([str(ROOT / "bin" / "generate"), str(folder), "5,6,7,8", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr
    ids = [int(x) for x in done.stdout.split()]
    tokens, margins = plain_greedy(pcfg, pw, [5, 6, 7, 8], 6)
    sure = next((i for i, m in enumerate(margins) if m < 1e-3), 6)
    assert ids[:4] == [5, 6, 7, 8] and ids[4:4 + sure] == tokens[:sure]
    a, b = sc.prompts(sc.ONLY_SHARED, [70, 9], seed=1)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:2], "want": []}],
              "end": []}]
    for i in range(7):
        live = [("a", a, 66 + i)] * (66 + i < len(a)) + [("b", b, 2 + i)]
        steps.append({"step": i + 1, "entries": [{"id": r, "tokens": [s[p]], "want": [0]} for r, s, p in live],
                      "end": [r for r, s, p in live if p + 1 == len(s)]})
    out = tmp_path / "out"
    run = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                          "--max-tokens", "79"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=900, env=dict(os.environ))
    assert run.returncode == 0, run.stderr
    assert run.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    ref = {"a": plain.forward(pcfg, pw, a), "b": plain.forward(pcfg, pw, b)}
    first = np.frombuffer((out / "0.f32").read_bytes(), dtype="<f4").reshape(2, -1)
    assert np.abs(first[1] - ref["a"][65]).max() / np.abs(ref["a"]).max() < 1e-4
    last = np.frombuffer((out / "7.f32").read_bytes(), dtype="<f4").reshape(1, -1)
    assert np.abs(last[0] - ref["b"][8]).max() / np.abs(ref["b"]).max() < 1e-4
