"""The kernels Gokezen added, each alone against float64: the matrix memory's recurrence (sizes on both sides of every
branch, runs of unequal length, a state carried from call to call, gates that saturate), RMS norm per head with a gate,
the clamped pair rule, the vector added to the stream, the router with its groups, and the experts' products over
sorted rows in both forms."""
import numpy as np
import pytest
import torch

import plain_gokezen as plain
from burn_transformers_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(DEV)


def rounded(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DT[dtype]).double().numpy()


def ints(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("heads, dim, vdim", [(3, 8, 5), (2, 32, 64), (1, 48, 72), (2, 100, 40), (1, 130, 300), (1, 256, 33)])
def test_memory_recurrence(dtype, heads, dim, vdim, chunked):
    rng = np.random.default_rng(dim * 7 + vdim)
    lengths = [1, 37, 16, 70]
    slots = [5, 0, 3, 2]
    cap = 7.0
    pad = 3
    width = 2 * heads * dim + heads * vdim + 2 * heads + pad
    offs = (pad, pad + heads * dim, pad + 2 * heads * dim, pad + 2 * heads * dim + heads * vdim,
            pad + 2 * heads * dim + heads * vdim + heads)
    i_bias, f_bias = rng.standard_normal(heads) * 0.5, rng.standard_normal(heads) + 3.0
    s = torch.zeros((6, heads, dim, vdim), device=DEV)
    n = torch.zeros((6, heads, dim), device=DEV)
    m = torch.zeros((6, heads), device=DEV)
    states = {}
    for call in range(2):      # the second call goes on from the first one's state
        total = sum(lengths)
        proj = rng.standard_normal((total, width))
        proj[:, offs[3]:offs[3] + 2 * heads] *= 6.0       # gates that reach the cap on both sides
        proj = rounded(proj, dtype)
        out = torch.full((total + 2, heads * vdim), 7.0, device=DEV)
        starts = np.concatenate([[0], np.cumsum(lengths)])
        scratch = None
        if chunked:
            need = kernels.mlstm_chunked_scratch_floats(total + 2, len(lengths), max(lengths), heads, dim, vdim)
            scratch = torch.full((need,), float("nan"), device=DEV)
        kernels.mlstm_scan(dev(proj, DT[dtype]), offs, dev(i_bias), dev(f_bias), cap, dim ** -0.5, s, n, m, ints(slots),
                           ints(starts), out, n_seqs=len(lengths), n_heads=heads, dim=dim, vdim=vdim, max_new=max(lengths),
                           scratch=scratch)
        got = out.cpu().double().numpy()
        assert np.all(got[total:] == 7.0)
        i_b32, f_b32 = i_bias.astype(np.float32).astype(np.float64), f_bias.astype(np.float32).astype(np.float64)
        for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            for a in range(heads):
                q = proj[lo:hi, offs[0] + a * dim:offs[0] + (a + 1) * dim] * dim ** -0.5
                k = proj[lo:hi, offs[1] + a * dim:offs[1] + (a + 1) * dim]
                v = proj[lo:hi, offs[2] + a * vdim:offs[2] + (a + 1) * vdim]
                ga, gb = plain.capped_gates(proj[lo:hi, offs[3] + a] + i_b32[a], proj[lo:hi, offs[4] + a] + f_b32[a], cap)
                want, states[(r, a)] = plain.memory_recurrence(q, k, v, ga, gb, states.get((r, a)))
                err = np.abs(got[lo:hi, a * vdim:(a + 1) * vdim] - want).max() / max(1.0, np.abs(want).max())
                assert err < 2e-4, (call, r, a, err)
    for (r, a), (S, nv, mv) in states.items():
        assert np.abs(s[slots[r], a].cpu().double().numpy() - S).max() < 2e-4 * max(1.0, np.abs(S).max())
        assert np.abs(n[slots[r], a].cpu().double().numpy() - nv).max() < 2e-4 * max(1.0, np.abs(nv).max())
        assert abs(float(m[slots[r], a]) - mv) < 1e-4
    assert float(s[1].abs().sum()) == 0 and float(s[4].abs().sum()) == 0      # slots of no sequence stay untouched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim", [(2, 32, 48), (1, 64, 64), (2, 100, 64), (3, 200, 32), (2, 8, 5), (1, 48, 72),
                                              (1, 130, 40)])
def test_memory_recurrence_with_the_norm_and_gate_inside(dtype, heads, dim, vdim):
    """Where a block holds a whole head, the token-by-token kernel norms each head's read-out and gates it itself."""
    rng = np.random.default_rng(dim + vdim)
    lengths, slots, cap, eps = [1, 20, 1, 7], [2, 0, 1, 3], 9.0, 1e-5
    width = 2 * heads * dim + 2 * heads * vdim + 2 * heads
    offs = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + 2 * heads * vdim, 2 * heads * dim + 2 * heads * vdim + heads)
    g_off = 2 * heads * dim + heads * vdim
    total = sum(lengths)
    proj = rounded(rng.standard_normal((total, width)), dtype)
    i_bias, f_bias = np.zeros(heads), np.full(heads, 2.0)
    weight = rounded(1.0 + 0.3 * rng.standard_normal(heads * vdim), "float32")
    s = torch.zeros((4, heads, dim, vdim), device=DEV)
    n = torch.zeros((4, heads, dim), device=DEV)
    m = torch.zeros((4, heads), device=DEV)
    out = torch.full((total, heads * vdim), 7.0, device=DEV)
    mixed = torch.full((total + 1, heads * vdim), 3.0, dtype=DT[dtype], device=DEV)
    starts = np.concatenate([[0], np.cumsum(lengths)])
    fused = kernels.mlstm_scan(dev(proj, DT[dtype]), offs, dev(i_bias), dev(f_bias), cap, dim ** -0.5, s, n, m, ints(slots),
                               ints(starts), out, n_seqs=len(lengths), n_heads=heads, dim=dim, vdim=vdim, max_new=max(lengths),
                               norm=(dev(weight), eps, g_off, mixed))
    assert fused == kernels.mlstm_scan_fuses(dim, vdim) == (vdim <= 32 or (vdim <= 64 and dim <= 128))
    if not fused:
        assert float((mixed.float() - 3.0).abs().sum()) == 0 and float((out - 7.0).abs().min()) > 0
        return
    got = mixed.float().cpu().double().numpy()
    assert np.all(got[total] == 3.0) and float((out - 7.0).abs().sum()) == 0
    for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
        for a in range(heads):
            ga, gb = plain.capped_gates(proj[lo:hi, offs[3] + a] + i_bias[a], proj[lo:hi, offs[4] + a] + f_bias[a], cap)
            o, _ = plain.memory_recurrence(proj[lo:hi, a * dim:(a + 1) * dim] * dim ** -0.5,
                                           proj[lo:hi, offs[1] + a * dim:offs[1] + (a + 1) * dim],
                                           proj[lo:hi, offs[2] + a * vdim:offs[2] + (a + 1) * vdim], ga, gb)
            want = (o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * weight[a * vdim:(a + 1) * vdim]
                    * plain.sigmoid(proj[lo:hi, g_off + a * vdim:g_off + (a + 1) * vdim]))
            err = np.abs(got[lo:hi, a * vdim:(a + 1) * vdim] - want).max() / np.abs(want).max()
            assert err < (2e-4 if dtype == "float32" else 1e-2), (r, a, err)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("long_run", [128, 130, 517, 2200])
def test_memory_recurrence_over_long_runs(long_run, chunked):
    """Runs longer than a chunk, forget gates close to one: what the first tokens wrote is still read at the end."""
    rng = np.random.default_rng(long_run)
    heads, dim, vdim, cap = 2, 24, 40, 12.0
    lengths = [long_run, 3, 65]
    width = 2 * heads * dim + heads * vdim + 2 * heads
    offs = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, 2 * heads * dim + heads * vdim + heads)
    total = sum(lengths)
    proj = rng.standard_normal((total, width))
    i_bias, f_bias = np.array([-1.0, 0.5]), np.array([6.0, 4.0])
    s = torch.zeros((3, heads, dim, vdim), device=DEV)
    n = torch.zeros((3, heads, dim), device=DEV)
    m = torch.zeros((3, heads), device=DEV)
    out = torch.zeros((total, heads * vdim), device=DEV)
    starts = np.concatenate([[0], np.cumsum(lengths)])
    scratch = None
    if chunked:
        scratch = torch.full((kernels.mlstm_chunked_scratch_floats(total, 3, max(lengths), heads, dim, vdim),), float("nan"),
                             device=DEV)
    kernels.mlstm_scan(dev(proj), offs, dev(i_bias), dev(f_bias), cap, dim ** -0.5, s, n, m, ints([2, 0, 1]), ints(starts),
                       out, n_seqs=3, n_heads=heads, dim=dim, vdim=vdim, max_new=max(lengths), scratch=scratch)
    got = out.cpu().double().numpy()
    proj = rounded(proj, "float32")
    for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
        for a in range(heads):
            ga, gb = plain.capped_gates(proj[lo:hi, offs[3] + a] + i_bias[a], proj[lo:hi, offs[4] + a] + f_bias[a], cap)
            want, (S, _, mv) = plain.memory_recurrence(proj[lo:hi, a * dim:(a + 1) * dim] * dim ** -0.5,
                                                       proj[lo:hi, offs[1] + a * dim:offs[1] + (a + 1) * dim],
                                                       proj[lo:hi, offs[2] + a * vdim:offs[2] + (a + 1) * vdim], ga, gb)
            assert np.abs(got[lo:hi, a * vdim:(a + 1) * vdim] - want).max() < 3e-4 * max(1.0, np.abs(want).max()), (r, a)
            assert np.abs(s[[2, 0, 1][r], a].cpu().double().numpy() - S).max() < 3e-4 * max(1.0, np.abs(S).max())


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups, width", [(1, 96), (4, 96), (3, 30), (5, 200), (1, 1000), (1, 1500), (2, 2400), (3, 600)])
def test_rms_norm_per_head_with_a_gate(out_dtype, groups, width):
    rng = np.random.default_rng(groups)
    rows = 9
    x, gate, weight = rng.standard_normal((rows, width)) * 3, rng.standard_normal((rows, width + 6)), rng.standard_normal(width)
    gate = rounded(gate, out_dtype)
    out = torch.full((rows + 1, width), 5.0, dtype=DT[out_dtype], device=DEV)
    kernels.rmsnorm(dev(x), dev(weight), out, 1e-5, n_rows=rows, gate=dev(gate, DT[out_dtype])[:, 4:4 + width], groups=groups)
    x32, w32 = rounded(x, "float32"), rounded(weight, "float32")
    per = x32.reshape(rows, groups, -1)
    want = (per / np.sqrt((per * per).mean(-1, keepdims=True) + 1e-5)).reshape(rows, width) * w32 * plain.sigmoid(gate[:, 4:4 + width])
    got = out.cpu().double().numpy()
    assert np.abs(got[:rows] - want).max() < (1e-5 if out_dtype == "float32" else 2e-2) * np.abs(want).max()
    assert np.all(got[rows] == 5.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner", [24, 20])
def test_clamped_pair_rule(dtype, inner):
    rng = np.random.default_rng(inner)
    x = rounded(rng.standard_normal((7, 2 * inner)) * 2.5, dtype)
    out = torch.zeros((7, inner), dtype=DT[dtype], device=DEV)
    kernels.gated_activation(dev(x, DT[dtype]), out, n_rows=7, activation="swish_clamp", limit=1.3)
    g, u = np.minimum(x[:, :inner], 1.3), np.clip(x[:, inner:], -1.3, 1.3)
    want = g * plain.sigmoid(1.702 * g) * (u + 1.0)
    assert np.abs(out.cpu().double().numpy() - want).max() < (1e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()


def test_vector_added_to_the_stream():
    x = torch.randn((11, 70), device=DEV)
    table = torch.randn((3, 70), device=DEV)
    want = x[:9] + table[2]
    kept = x[9:].clone()
    kernels.add_vector(x, table[2], n_rows=9)
    assert torch.equal(x[:9], want) and torch.equal(x[9:], kept)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, groups, keep", [(12, 3, 3, 2), (16, 4, 2, 1), (5, 2, 1, 1), (64, 6, 8, 3), (7, 7, 1, 1),
                                                        (40, 1, 40, 1), (6, 2, 6, 2)])
def test_router(dtype, experts, top, groups, keep):
    rng = np.random.default_rng(experts * 10 + top)
    tokens, width = 77, 50
    x, router = rounded(rng.standard_normal((tokens, width)), dtype), rounded(rng.standard_normal((experts, width)) * 0.3, dtype)
    ids = torch.full((tokens + 1, top), -1, dtype=torch.int32, device=DEV)
    weights = torch.zeros((tokens + 1, top), device=DEV)
    kernels.moe_route(dev(x, DT[dtype]), dev(router, DT[dtype]), ids, weights, n_tokens=tokens, top=top, n_groups=groups,
                      keep=keep, scale=1.7)
    want_ids, want_w = plain.route(x, router, {"experts": experts, "top": top, "scale": 1.7,
                                               "groups": {"count": groups, "keep": keep}})
    got_ids = ids.cpu().numpy()
    assert np.all(got_ids[tokens] == -1)
    scores = np.sort(plain.sigmoid(x @ router.T), axis=1)
    close = np.min(np.diff(scores, axis=1), axis=1) < 1e-6        # (a choice between two equal scores proves nothing)
    assert close.sum() < 5
    assert np.array_equal(got_ids[:tokens][~close], want_ids[~close])
    assert np.abs(weights.cpu().double().numpy()[:tokens][~close] - want_w[~close]).max() < 1e-5


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("tokens, width, inner, experts, top", [(150, 64, 48, 6, 2), (9, 40, 24, 16, 4), (70, 72, 20, 3, 3),
                                                               (1, 32, 16, 8, 1), (300, 96, 80, 5, 2)])
def test_experts_over_sorted_rows(dtype, tensor_cores, tokens, width, inner, experts, top):
    rng = np.random.default_rng(tokens + experts)
    x = rounded(rng.standard_normal((tokens, width)), dtype)
    w_in = rounded(rng.standard_normal((experts, 2 * inner, width)) * width ** -0.5, dtype)
    w_out = rounded(rng.standard_normal((experts, width, inner)) * inner ** -0.5, dtype)
    # (with many tokens expert 1 gets no row at all)
    pool = np.array([e for e in range(experts) if not (tokens > 100 and e == 1)])
    chosen = np.stack([rng.permutation(pool)[:top] for _ in range(tokens)])
    pair_w = rng.random((tokens, top)) + 0.1
    pairs = tokens * top
    ids = dev(chosen, torch.int32)
    offsets, tile_first = torch.zeros(experts + 1, dtype=torch.int32, device=DEV), torch.zeros(experts + 1, dtype=torch.int32, device=DEV)
    order, place = torch.zeros(pairs, dtype=torch.int32, device=DEV), torch.zeros(pairs, dtype=torch.int32, device=DEV)
    kernels.moe_sort(ids, offsets, tile_first, order, place, pairs=pairs, n_experts=experts)
    counts = np.bincount(chosen.reshape(-1), minlength=experts)
    assert np.array_equal(offsets.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(tile_first.cpu().numpy(), np.concatenate([[0], np.cumsum(-(-counts // 32))]))
    o, p = order.cpu().numpy(), place.cpu().numpy()
    assert sorted(o) == list(range(pairs)) and np.array_equal(p[o], np.arange(pairs))
    assert np.array_equal(chosen.reshape(-1)[o], np.repeat(np.arange(experts), counts))
    hidden = torch.zeros((pairs + 1, inner), dtype=DT[dtype], device=DEV)
    kernels.moe_expert(True, dev(x, DT[dtype]), dev(w_in, DT[dtype]), hidden, offsets, tile_first, order, None, pairs=pairs,
                       top=top, activation="swish_clamp", limit=1.1, tensor_cores=tensor_cores)
    part = torch.zeros((pairs + 1, width), device=DEV)
    weights = dev(pair_w)
    kernels.moe_expert(False, hidden, dev(w_out, DT[dtype]), part, offsets, tile_first, order, weights, pairs=pairs, top=top,
                       tensor_cores=tensor_cores)
    stream = torch.ones((tokens, width), device=DEV)
    kernels.moe_combine(part, place, stream, n_tokens=tokens, top=top)
    assert float(hidden[pairs].abs().sum()) == 0 and float(part[pairs].abs().sum()) == 0
    want = np.ones((tokens, width))
    pair_w32 = rounded(pair_w, "float32")
    got_hidden = hidden.cpu().double().numpy()
    for t in range(tokens):
        for j, e in enumerate(chosen[t]):
            g, u = np.minimum(w_in[e, :inner] @ x[t], 1.1), np.clip(w_in[e, inner:] @ x[t], -1.1, 1.1)
            h = g * plain.sigmoid(1.702 * g) * (u + 1.0)
            tol = 1e-5 if dtype == "float32" else 2e-2
            assert np.abs(got_hidden[p[t * top + j]] - h).max() < tol * max(1.0, np.abs(h).max())
            want[t] += pair_w32[t, j] * (w_out[e] @ got_hidden[p[t * top + j]])
    assert np.abs(stream.cpu().double().numpy() - want).max() < 2e-5 * np.abs(want).max()
