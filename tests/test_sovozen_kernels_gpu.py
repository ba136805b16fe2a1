"""The kernels of the latent attention, the decayed recurrence and the row-wise steps, each alone against NumPy
float64, at sizes the models of the other tests do not have, with keys planted where a fault would hide."""
import numpy as np
import pytest
import torch

import plain_sovozen as plain
from burn_transformers_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)]


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=torch.float64).to(dtype).to(DEV)


def host(t):
    return t.detach().double().cpu().numpy()


def rel(got, want):
    return float(np.abs(got - want).max() / max(1e-30, np.abs(want).max()))


@pytest.mark.parametrize("dtype, tol", DTYPES)
def test_rotation_of_a_slice_of_every_head(dtype, tol):
    rng = np.random.default_rng(0)
    n, heads, plain_dims, length, dims = 7, 3, 5, 10, 6
    freq = torch.tensor([50.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    rows = dev(rng.standard_normal((n, heads * (plain_dims + length) + 3)), dtype)
    positions = torch.tensor([0, 1, 2, 700, 64, 63, 5], dtype=torch.int32, device=DEV)
    src = rows[:, :heads * (plain_dims + length)].view(n, heads, plain_dims + length)[:, :, plain_dims:]
    out = torch.full((n, heads, length + 2), 9.0, dtype=dtype, device=DEV)
    kernels.rotary_interleaved(src, out[:, :, :length], positions, freq, n_tokens=n, dims=dims)
    want = plain.rotate_interleaved(host(src), host(positions), dims, 50.0)
    assert rel(host(out[:, :, :length]), want) < tol
    assert bool((out[:, :, length:] == 9.0).all())
    before = host(src).copy()
    kernels.rotary_interleaved(src, src, positions, freq, n_tokens=n, dims=dims)          # in place
    assert rel(host(src), plain.rotate_interleaved(before, host(positions), dims, 50.0)) < tol


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("gated", [False, True])
def test_rms_norm_with_and_without_a_gate(dtype, tol, gated):
    rng = np.random.default_rng(1)
    n, width = 5, 77
    x = dev(rng.standard_normal((n, width)) * 3.0)
    gate_rows = dev(rng.standard_normal((n, width + 9)), dtype)
    weight = dev(1.0 + 0.3 * rng.standard_normal(width))
    out = torch.zeros((n + 2, width), dtype=dtype, device=DEV)
    kernels.rmsnorm(x, weight, out, 1e-3, n_rows=n, gate=gate_rows[:, 9:] if gated else None)
    want = plain.rms_norm(host(x), host(weight), 1e-3)
    if gated:
        want = want * plain.sigmoid(host(gate_rows[:, 9:]))
    assert rel(host(out[:n]), want) < tol and bool((out[n:] == 0).all())


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("inner", [50, 64, 200])
def test_gated_activation(dtype, tol, inner):
    rng = np.random.default_rng(2)
    n = 6
    x = dev(rng.standard_normal((n, 2 * inner)) * 2.0, dtype)
    out = torch.zeros((n + 1, inner), dtype=dtype, device=DEV)
    kernels.gated_activation(x, out, n_rows=n, activation="gelu_new")
    xs = host(x)
    assert rel(host(out[:n]), plain.gelu_tanh(xs[:, :inner]) * xs[:, inner:]) < tol and bool((out[n:] == 0).all())


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("n, heads, k, width, skip", [(19, 3, 21, 13, 4), (70, 3, 64, 72, 8), (5, 2, 256, 64, 0),
                                                      (130, 5, 40, 24, 16), (64, 1, 72, 136, 8)])
def test_products_per_head_with_a_gate(dtype, tol, n, heads, k, width, skip):
    """Odd sizes take the multiply-add kernel; in bfloat16, operands on 16-byte boundaries take the tensor cores."""
    rng = np.random.default_rng(3)
    a_rows = dev(rng.standard_normal((n, heads * (k + skip))), dtype)
    a = a_rows.view(n, heads, k + skip)[:, :, skip:]
    w = dev(rng.standard_normal((heads, k, width)) / np.sqrt(k), dtype)
    gate = dev(rng.standard_normal((n, heads, width)), dtype)
    out = torch.zeros((n + 1, heads, width), dtype=dtype, device=DEV)
    kernels.head_linear(a, w, out, n_tokens=n)
    want = np.einsum("thk,hkj->thj", host(a), host(w))
    assert rel(host(out[:n]), want) < tol and bool((out[n:] == 0).all())
    kernels.head_linear(a, w, out, n_tokens=n, gate=gate)
    assert rel(host(out[:n]), want * plain.sigmoid(host(gate))) < tol


def pages_for(lengths, rng):
    """A page table that scatters every sequence's pages over the pool."""
    counts = [-(-n // 64) for n in lengths]
    order = rng.permutation(sum(counts) + 3)
    table = np.zeros((len(lengths), max(counts)), dtype=np.int32)
    at = 0
    for s, c in enumerate(counts):
        table[s, :c] = order[at:at + c]
        at += c
    return table, len(order)


def latent_reference(q, rows, rank, scale, sink, past, seq_of, pos_of):
    """q [tokens, heads, rank + rot] against rows[seq] [length, rank + rot]: softmax with a sink over the keys up to
    each token's own position, mixing the first `rank` channels."""
    out = np.zeros((q.shape[0], q.shape[1], rank))
    for t in range(q.shape[0]):
        keys = rows[seq_of[t]][:pos_of[t] + 1]
        for h in range(q.shape[1]):
            scores = (keys @ q[t, h]) * scale
            out[t, h] = plain.sink_softmax_mix(scores[None, :], sink[h] if sink is not None else -np.inf, keys[:, :rank])[0]
    return out


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("heads, rank, rot, splits", [(3, 24, 6, 1), (5, 72, 0, 3), (40, 160, 8, 1), (2, 300, 4, 7),
                                                      (8, 32, 8, 2), (4, 64, 16, 1), (12, 256, 32, 1), (70, 128, 8, 2),
                                                      (16, 512, 64, 3)])
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_latent_attention_over_scattered_pages(dtype, tol, heads, rank, rot, splits, tensor_cores):
    """Prompts that continue cached sequences and sequences of one new token, with and without a sink, any number of
    splits: every row against the plain softmax.  bfloat16 runs both of its kernels (tensor cores where the shape is
    one of theirs, and the multiply-add kernel)."""
    if dtype == torch.float32 and not tensor_cores:
        pytest.skip("32-bit has one kernel")
    rng = np.random.default_rng(rank)
    dk = rank + rot
    lengths, new = [130, 64, 33, 1], [66, 1, 33, 1]          # the sequences' lengths after the step; their new tokens
    table, n_pages = pages_for(lengths, rng)
    pool = torch.zeros((n_pages, 64, dk), dtype=dtype, device=DEV)
    rows = [np.asarray(host(dev(rng.standard_normal((n, dk)) * 0.7, dtype))) for n in lengths]
    for s, r in enumerate(rows):
        for p in range(len(r)):
            pool[table[s, p // 64], p % 64] = dev(r[p], dtype)
    n = sum(new)
    q = dev(rng.standard_normal((n, heads * dk)) * 0.7, dtype)
    seq_start = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    past = np.asarray([l - m for l, m in zip(lengths, new)], dtype=np.int32)
    seq_of = [s for s, m in enumerate(new) for _ in range(m)]
    pos_of = [past[s] + i for s, m in enumerate(new) for i in range(m)]
    sink = rng.standard_normal(heads) * 2.0
    for use_sink in (True, False):
        out = torch.zeros((n + 1, heads * rank), dtype=dtype, device=DEV)
        scratch = torch.zeros(max(1, kernels.latent_attention_scratch_floats(n, heads, rank, splits)), device=DEV)
        kernels.latent_attention(q, out, pool, torch.tensor(table, device=DEV), table.shape[1],
                                 torch.tensor(seq_start, device=DEV), torch.tensor(past, device=DEV), n_tokens=n,
                                 n_seqs=len(new), max_new=max(new), n_heads=heads, rank=rank, rot=rot, scale=0.21,
                                 sink=dev(sink) if use_sink else None, n_splits=splits, scratch=scratch,
                                 tensor_cores=tensor_cores)
        want = latent_reference(host(q).reshape(n, heads, dk), rows, rank, 0.21, sink if use_sink else None, past, seq_of,
                                pos_of)
        assert rel(host(out[:n]).reshape(n, heads, rank), want) < tol
        assert bool((out[n:] == 0).all())


@pytest.mark.parametrize("target", [0, 31, 32, 63, 64, 65, 500, 699])
@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("dtype, close", [(torch.float32, 1e-3), (torch.bfloat16, 2e-2)])
def test_one_key_among_hundreds_carries_the_row(target, splits, dtype, close):
    """A query that matches one far key and nothing else must return that key's latent: a key that is skipped, read from
    a wrong page or masked by mistake shows at once.  The same key planted one position AFTER the query must stay
    unseen."""
    rng = np.random.default_rng(7)
    rank, rot, heads, length = 24, 8, 2, 700
    dk = rank + rot
    rows = rng.standard_normal((length, dk)) * 0.05
    rows[target] = 0.0
    rows[target, rank:] = 3.0                       # loud in the shared rotated part
    rows[target, :rank] = np.linspace(-1, 1, rank)
    table, n_pages = pages_for([length], rng)
    pool = torch.zeros((n_pages, 64, dk), dtype=dtype, device=DEV)
    for p in range(length):
        pool[table[0, p // 64], p % 64] = dev(rows[p], dtype)
    q = np.zeros((2, heads, dk))
    q[:, :, rank:] = 3.0
    # two query tokens in one step: one right before the target (must not see it), the last one of the sequence
    first_pos = max(0, target - 1)
    out = torch.zeros((2, heads * rank), dtype=dtype, device=DEV)
    scratch = torch.zeros(max(1, kernels.latent_attention_scratch_floats(2, heads, rank, splits)), device=DEV)
    for pos in (first_pos, length - 1):
        kernels.latent_attention(dev(q.reshape(2, heads * dk), dtype), out, pool, torch.tensor(table, device=DEV), table.shape[1],
                                 torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                 torch.tensor([pos], dtype=torch.int32, device=DEV), n_tokens=1, n_seqs=1, max_new=1,
                                 n_heads=heads, rank=rank, rot=rot, scale=1.0, sink=None, n_splits=splits, scratch=scratch)
        got = host(out[0]).reshape(heads, rank)
        sees = pos >= target
        if sees:
            assert np.abs(got - rows[target, :rank]).max() < close, (pos, target)
        else:
            assert np.abs(got).max() < 0.2, (pos, target)          # only quiet keys: nothing near the planted latent
    # a sink far above every score takes all the weight: the output vanishes
    kernels.latent_attention(dev(q.reshape(2, heads * dk), dtype), out, pool, torch.tensor(table, device=DEV), table.shape[1],
                             torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                             torch.tensor([length - 1], dtype=torch.int32, device=DEV), n_tokens=1, n_seqs=1, max_new=1,
                             n_heads=heads, rank=rank, rot=rot, scale=1.0, sink=dev([200.0, -200.0]), n_splits=splits,
                             scratch=scratch)
    got = host(out[0]).reshape(heads, rank)
    assert np.abs(got[0]).max() < 1e-6 and np.abs(got[1] - rows[target, :rank]).max() < close


@pytest.mark.parametrize("dtype, tol", DTYPES)
def test_latent_rows_are_normed_turned_and_filed(dtype, tol):
    rng = np.random.default_rng(9)
    rank, rot, dims, n = 20, 10, 6, 5
    src_rows = dev(rng.standard_normal((n, 7 + rank + rot)) * 2.0, dtype)
    weight = dev(1.0 + 0.2 * rng.standard_normal(rank))
    freq = torch.tensor([30.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    positions = np.asarray([63, 64, 65, 0, 130], dtype=np.int32)
    token_seq = np.asarray([0, 0, 0, 1, 1], dtype=np.int32)
    table = np.asarray([[4, 1, 9], [2, 7, 5]], dtype=np.int32)
    pool = torch.full((10, 64, rank + rot), 5.0, dtype=dtype, device=DEV)
    kernels.latent_append(src_rows[:, 7:], weight, 1e-4, torch.tensor(positions, device=DEV),
                          torch.tensor(token_seq, device=DEV), freq, dims, torch.tensor(table, device=DEV), 3, pool, n,
                          rank, rot)
    src = host(src_rows[:, 7:])
    want_c = plain.rms_norm(src[:, :rank], host(weight), 1e-4)
    want_r = plain.rotate_interleaved(src[:, rank:], positions, dims, 30.0)
    written = torch.zeros_like(pool, dtype=torch.bool)
    for t in range(n):
        page, at = table[token_seq[t], positions[t] // 64], positions[t] % 64
        got = host(pool[page, at])
        assert rel(got[:rank], want_c[t]) < tol and rel(got[rank:], want_r[t]) < tol
        written[page, at] = True
    assert bool((pool[~written] == 5.0).all())


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("heads, dim, vdim", [(2, 16, 24), (1, 40, 8), (3, 128, 70), (2, 200, 33)])
@pytest.mark.parametrize("steps", [[[40, 1, 17], [2, 33, 1], [1, 1, 1]], [[150, 64, 65], [70, 1, 129], [1, 1, 1]]])
def test_recurrence_carries_its_state_from_step_to_step(dtype, tol, heads, dim, vdim, steps):
    """Three sequences in scattered slots: a prompt, then a portion, then one token each; every output against the plain
    recurrence over the whole sequences.  Runs of more than 64 tokens take the chunked form (whole chunks, a ragged last
    chunk, a state carried in from the step before); shorter ones go token by token."""
    rng = np.random.default_rng(dim)
    decay = rng.uniform(0.5, 1.0, heads)
    slots = np.asarray([5, 0, 3], dtype=np.int32)
    state = torch.zeros((7, heads, dim, vdim), device=DEV)
    state[1] = 4.0                                              # a slot of another sequence: must stay as it is
    width = 2 * heads * dim + heads * vdim + 5
    totals = np.sum(steps, axis=0)
    rows = [np.asarray(host(dev(rng.standard_normal((n, width)), dtype))) for n in totals]
    want = []
    for r in rows:
        q = plain.silu(r[:, 3:3 + heads * dim]).reshape(-1, heads, dim)
        k = plain.silu(r[:, 3 + heads * dim:3 + 2 * heads * dim]).reshape(-1, heads, dim)
        v = plain.silu(r[:, 5 + 2 * heads * dim:]).reshape(-1, heads, vdim)
        o = np.zeros((len(r), heads, vdim))
        for h in range(heads):
            s = np.zeros((dim, vdim))
            for t in range(len(r)):
                s = decay[h] * s + np.outer(k[t, h], v[t, h])
                o[t, h] = s.T @ q[t, h]
        want.append(o.reshape(len(r), heads * vdim))
    fed = [0, 0, 0]
    for step in steps:
        proj = dev(np.concatenate([rows[i][fed[i]:fed[i] + m] for i, m in enumerate(step)]), dtype)
        n = sum(step)
        out = torch.zeros((n + 1, heads * vdim), device=DEV)
        seq_start = np.concatenate([[0], np.cumsum(step)]).astype(np.int32)
        scratch = torch.zeros(max(1, kernels.lightning_chunked_scratch_floats(3, max(step), heads, dim, vdim)), device=DEV)
        kernels.lightning_scan(proj, 3, 3 + heads * dim, 5 + 2 * heads * dim, state, torch.tensor(slots, device=DEV),
                               torch.tensor(seq_start, device=DEV), dev(decay), out, n_seqs=3, n_heads=heads, dim=dim,
                               vdim=vdim, max_new=max(step), scratch=scratch)
        expect = np.concatenate([want[i][fed[i]:fed[i] + m] for i, m in enumerate(step)])
        assert rel(host(out[:n]), expect) < tol and bool((out[n:] == 0).all())
        fed = [f + m for f, m in zip(fed, step)]
    assert bool((state[1] == 4.0).all()) and bool((state[[2, 4, 6]] == 0).all())


@pytest.mark.parametrize("heads, dq, dv", [(3, 48, 40), (2, 96, 64), (1, 136, 128), (5, 16, 8)])
@pytest.mark.parametrize("with_sink, with_gate", [(True, True), (False, False)])
def test_attention_of_fresh_prompts_with_a_sink_and_a_gate(heads, dq, dv, with_sink, with_gate):
    """Sequences of 1, 33, 64, 65 and 200 tokens in one call, heads as strided views of wider rows: every row against the
    plain softmax over the keys up to its own position."""
    rng = np.random.default_rng(dq)
    lengths = [65, 1, 200, 33, 64]
    n = sum(lengths)
    wide = dev(rng.standard_normal((n, heads * (dq + 8) + 16)) * 0.6, torch.bfloat16)
    q = wide[:, 16:].view(n, heads, dq + 8)[:, :, 8:]
    k = dev(rng.standard_normal((n, heads, dq)) * 0.6, torch.bfloat16)
    v = dev(rng.standard_normal((n, heads, dv)), torch.bfloat16)
    gate = dev(rng.standard_normal((n, heads, dv)), torch.bfloat16) if with_gate else None
    sink = rng.standard_normal(heads) * 2.0
    out = torch.zeros((n + 1, heads, dv), dtype=torch.bfloat16, device=DEV)
    seq_start = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    assert kernels.sink_attention_supports(q, k, v, gate, out[:n])
    kernels.sink_attention(q, k, v, out[:n], torch.tensor(seq_start, device=DEV), n_seqs=len(lengths),
                           max_new=max(lengths), scale=0.17, sink=dev(sink) if with_sink else None, gate=gate)
    qh, kh, vh = host(q), host(k), host(v)
    want = np.zeros((n, heads, dv))
    for s, length in enumerate(lengths):
        lo = seq_start[s]
        for h in range(heads):
            scores = (qh[lo:lo + length, h] @ kh[lo:lo + length, h].T) * 0.17
            scores = np.where(np.tril(np.ones((length, length), dtype=bool)), scores, -np.inf)
            want[lo:lo + length, h] = plain.sink_softmax_mix(scores, sink[h] if with_sink else -np.inf, vh[lo:lo + length, h])
    if with_gate:
        want = want * plain.sigmoid(host(gate))
    assert rel(host(out[:n]), want) < 2e-2 and bool((out[n:] == 0).all())


def test_gather_of_the_steps_own_latent_rows():
    rng = np.random.default_rng(4)
    dk = 40
    pool = dev(rng.standard_normal((9, 64, dk)), torch.bfloat16)
    positions = torch.tensor([0, 63, 64, 130, 5], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 8, 0], [1, 4, 6]], dtype=torch.int32, device=DEV)
    rows = torch.zeros((6, dk), dtype=torch.bfloat16, device=DEV)
    kernels.latent_gather(pool, positions, token_seq, table, 3, rows, n_tokens=5)
    want = torch.stack([pool[3, 0], pool[3, 63], pool[8, 0], pool[6, 2], pool[1, 5]])
    assert torch.equal(rows[:5], want) and bool((rows[5] == 0).all())


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("owns", [True, False])
def test_fused_steps_before_the_attention_of_few_tokens(dtype, tol, owns):
    """One launch: the query carried into the latent space, its rotated part turned, and (for a layer with a latent of its
    own) the token's latent row normed, turned and filed."""
    rng = np.random.default_rng(12)
    n, heads, dim, rank, rot, dims = 5, 3, 20, 24, 10, 6
    q_off, lat_off = 0, heads * (dim + rot) + 7
    proj = dev(rng.standard_normal((n, lat_off + rank + rot + 3)), dtype)
    uk = dev(rng.standard_normal((heads, dim, rank)) / np.sqrt(dim), dtype)
    weight = dev(1.0 + 0.2 * rng.standard_normal(rank))
    freq = torch.tensor([30.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    positions = np.asarray([63, 64, 200, 0, 7], dtype=np.int32)
    token_seq = np.asarray([0, 1, 2, 3, 4], dtype=np.int32)
    table = rng.permutation(20).reshape(5, 4).astype(np.int32)
    pool = torch.full((20, 64, rank + rot), 5.0, dtype=dtype, device=DEV)
    q_latent = torch.zeros((n + 1, heads * (rank + rot)), dtype=dtype, device=DEV)
    kernels.latent_decode_prep(proj, q_off, lat_off, uk, weight if owns else None, 1e-4, torch.tensor(positions, device=DEV),
                               torch.tensor(token_seq, device=DEV), freq, dims, torch.tensor(table, device=DEV), 4, pool,
                               q_latent, n_tokens=n, n_heads=heads, dim=dim, rank=rank, rot=rot, owns=owns)
    p = host(proj)
    q = p[:, :heads * (dim + rot)].reshape(n, heads, dim + rot)
    want = np.concatenate([np.einsum("thd,hdr->thr", q[:, :, :dim], host(uk)),
                           plain.rotate_interleaved(q[:, :, dim:], positions, dims, 30.0)], axis=-1)
    assert rel(host(q_latent[:n]).reshape(n, heads, rank + rot), want) < tol and bool((q_latent[n:] == 0).all())
    written = torch.zeros_like(pool, dtype=torch.bool)
    if owns:
        lat = p[:, lat_off:lat_off + rank + rot]
        want_c = plain.rms_norm(lat[:, :rank], host(weight), 1e-4)
        want_r = plain.rotate_interleaved(lat[:, rank:], positions, dims, 30.0)
        for t in range(n):
            page, at = table[token_seq[t], positions[t] // 64], positions[t] % 64
            got = host(pool[page, at])
            assert rel(got[:rank], want_c[t]) < tol and rel(got[rank:], want_r[t]) < tol
            written[page, at] = True
    assert bool((pool[~written] == 5.0).all())


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("splits", [1, 5, 40])
def test_fused_steps_after_the_attention_of_few_tokens(dtype, tol, splits):
    """One launch: the splits' partial results joined (or the single result read), times W_uv per head, times the gate."""
    rng = np.random.default_rng(13)
    n, heads, rank, vdim = 4, 3, 40, 24
    uv = dev(rng.standard_normal((heads, rank, vdim)) / np.sqrt(rank), dtype)
    gate_rows = dev(rng.standard_normal((n, heads * vdim + 6)), dtype)
    out = torch.zeros((n + 1, heads * vdim), dtype=dtype, device=DEV)
    if splits == 1:
        mixed_latent = dev(rng.standard_normal((n, heads * rank)), dtype)
        merged = host(mixed_latent).reshape(n, heads, rank)
        kernels.latent_decode_finish(uv, out, n_tokens=n, n_splits=1, mixed_latent=mixed_latent, gate=gate_rows[:, 6:])
    else:
        sums = rng.standard_normal((n, heads, splits, rank))
        maxima = rng.standard_normal((n, heads, splits)) * 3.0
        maxima[:, :, 1] = -np.inf                       # a split that saw no key
        sums[:, :, 1] = 0.0
        denoms = rng.uniform(0.5, 2.0, (n, heads, splits))
        denoms[:, :, 1] = 0.0
        part = np.concatenate([sums, maxima[..., None], denoms[..., None]], axis=-1)
        w = np.where(np.isfinite(maxima), np.exp(maxima - maxima.max(axis=-1, keepdims=True)), 0.0)
        merged = (sums * w[..., None]).sum(axis=2) / (denoms * w).sum(axis=2)[..., None]
        kernels.latent_decode_finish(uv, out, n_tokens=n, n_splits=splits, scratch=dev(part.reshape(-1)),
                                     gate=gate_rows[:, 6:])
    want = np.einsum("thr,hrv->thv", merged, host(uv)) * plain.sigmoid(host(gate_rows[:, 6:]).reshape(n, heads, vdim))
    assert rel(host(out[:n]).reshape(n, heads, vdim), want) < tol and bool((out[n:] == 0).all())
