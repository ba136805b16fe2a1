"""Gokezen, written plainly: NumPy, float64, whole sequences, no cache, one function per mechanism.

This is the oracle of the Gokezen tests.  It shares no code with the library: it reads a configuration as a plain
dictionary and the weights as a dictionary of arrays under their checkpoint names, and loops over tokens, heads and
experts where the library has kernels.

The model: token embedding plus a learned position vector; layers in which ONE RMS norm feeds a mixer and a
feed-forward whose results are both added to the stream; the mixer is a windowed softmax attention with shared key
heads beside a matrix-memory recurrence (exponential input gate, sigmoid forget gate, a running maximum that keeps the
exponentials in range), each with a weight; the feed-forward is dense and gated, or routed experts with a shared one;
a run of layers may be repeated with the same weights, each pass opened by a learned vector; RMS norm and a readout
with the embedding table.
"""
from __future__ import annotations

import numpy as np


def rms_norm(x, weight, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def window_attention(h, w, prefix, c):
    """Softmax attention in which token i sees tokens i - window + 1 .. i; query head a reads key head a // (H / G)."""
    T = h.shape[0]
    H, G, dim, vdim, window = c["heads"], c["kv_heads"], c["dim"], c["vdim"], c["mask"]["size"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim)
    k = (h @ w[prefix + "k"].T).reshape(T, G, dim)
    v = (h @ w[prefix + "v"].T).reshape(T, G, vdim)
    out = np.zeros((T, H, vdim))
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, a]) * c["scale"]
            p = np.exp(s - s.max())
            out[i, a] = (p / p.sum()) @ v[lo:i + 1, g]
    return out.reshape(T, H * vdim) @ w[prefix + "o"].T


def memory_recurrence(q, k, v, a, b, state=None):
    """One head: q, k [T, dim], v [T, vdim], log gates a (input) and b (forget) [T]; state (S, n, m) or None for a
    sequence that starts.  Returns (o [T, vdim], state after the last token).

        m_t = max(b_t + m_(t-1), a_t)
        S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T       (n_t the same with k_t alone)
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)"""
    T, dim = q.shape
    S, n, m = (np.zeros((dim, v.shape[1])), np.zeros(dim), 0.0) if state is None else state
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        m_new = max(b[t] + m, a[t])
        keep, take = np.exp(b[t] + m - m_new), np.exp(a[t] - m_new)
        S = keep * S + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        out[t] = S.T @ q[t] / (max(abs(n @ q[t]), np.exp(-m)) + 1e-6)
    return out, (S, n, m)


def capped_gates(x_i, x_f, cap):
    """Log input gate and log forget gate from their pre-activations (biases already added)."""
    return cap * np.tanh(x_i / cap), log_sigmoid(cap * np.tanh(x_f / cap))


def matrix_memory(h, w, prefix, c, eps):
    """Per head a matrix S (dim x vdim), a vector n (dim) and a running maximum m, all zero before the first token
    (memory_recurrence), read by q = W_q h * dim^-1/2; then each head's o_t over its own root mean square, the heads side
    by side times a weight and a sigmoid gate, then W_o."""
    T = h.shape[0]
    H, dim, vdim, cap = c["heads"], c["dim"], c["vdim"], c["gate_cap"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w[prefix + "k"].T).reshape(T, H, dim)
    v = (h @ w[prefix + "v"].T).reshape(T, H, vdim)
    gi, gf = capped_gates(h @ w[prefix + "i"].T + w[prefix + "i.b"], h @ w[prefix + "f"].T + w[prefix + "f.b"], cap)
    out = np.zeros((T, H, vdim))
    for a in range(H):
        o, _ = memory_recurrence(q[:, a], k[:, a], v[:, a], gi[:, a], gf[:, a])
        out[:, a] = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps)
    flat = out.reshape(T, H * vdim) * w[prefix + "norm"] * sigmoid(h @ w[prefix + "g"].T)
    return flat @ w[prefix + "o"].T


def side_by_side(h, w, prefix, c, eps):
    left = window_attention(h, w, prefix + "left.", c["left"])
    right = matrix_memory(h, w, prefix + "right.", c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def dense_feed_forward(h, w, prefix):
    return (gelu_tanh(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def clamped_expert(h, w, prefix, limit):
    g = np.minimum(h @ w[prefix + "gate"].T, limit)
    u = np.clip(h @ w[prefix + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def route(h, router, c, margins=None):
    """(chosen experts [T, top], their weights [T, top]) of sigmoid scores, experts of the best groups only.  `margins`
    (an array [T]) is lowered, per token, to the smallest gap by which a group or an expert was preferred to the best
    one that was left out: where it is tiny, rounding decides the choice and a comparison proves nothing."""
    E, top = c["experts"], c["top"]
    groups = c.get("groups") or {"count": 1, "keep": 1}
    scores = sigmoid(h @ router.T)
    T = h.shape[0]
    chosen = np.zeros((T, top), dtype=np.int64)
    weights = np.zeros((T, top))
    size = E // groups["count"]
    for t in range(T):
        by_group = scores[t].reshape(groups["count"], size)
        group_score = np.sort(by_group, axis=1)[:, ::-1][:, :2].sum(axis=1)
        kept = np.argsort(-group_score, kind="stable")[:groups["keep"]]
        allowed = np.full(E, -np.inf)
        for g in kept:
            allowed[g * size:(g + 1) * size] = scores[t, g * size:(g + 1) * size]
        ranked = np.argsort(-allowed, kind="stable")
        chosen[t] = ranked[:top]
        if margins is not None:
            by_score = np.sort(group_score)[::-1]
            if groups["keep"] < groups["count"]:
                margins[t] = min(margins[t], by_score[groups["keep"] - 1] - by_score[groups["keep"]])
            if top < len(kept) * size:
                margins[t] = min(margins[t], allowed[ranked[top - 1]] - allowed[ranked[top]])
        picked = scores[t, chosen[t]]
        weights[t] = picked / (picked.sum() + 1e-20) * c["scale"]
    return chosen, weights


def routed_feed_forward(h, w, prefix, c, margins=None):
    chosen, weights = route(h, w[prefix + "router"], c["router"], margins)
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t], weights[t]):
            out[t] += weight * clamped_expert(h[t:t + 1], w, f"{prefix}e{e}.", c["expert"]["limit"])[0]
    if c.get("shared") is not None:
        out += clamped_expert(h, w, prefix + "shared.", c["shared"]["limit"])
    return out


def feed_forward(h, w, prefix, c, margins=None):
    if c is None:
        return 0.0
    return dense_feed_forward(h, w, prefix) if c["kind"] == "dense" else routed_feed_forward(h, w, prefix, c, margins)


def run_order(config):
    """[(layer, pass number or None when the layer opens no pass)]: the layers of the repeated run `times` times."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(config, w, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run).  `margins`: see route."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][np.asarray(tokens)] + w["pos"][:T]
    layers = []
    for i, opens in run_order(config):
        layer = config["layers"][i]
        if opens is not None:
            x = x + w["loop.step"][opens]
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        x = x + (side_by_side(h, w, f"l{i}.mix.", layer["mixer"], eps) + feed_forward(h, w, f"l{i}.mlp.", layer.get("mlp"), margins))
        layers.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, np.stack(layers)) if return_layers else logits
