"""A plain, slow Sovozen in NumPy float64: whole sequences, no cache, one function per mechanism.

The oracle of the Sovozen tests.  It shares no code with the library: it takes a configuration as a plain
dictionary (the keys of config.json) and the weights as a dictionary of float64 arrays by checkpoint name.

Notation: h is a [T, width] block of rows (one sequence, positions 0..T-1), W x means x @ W.T for a weight stored
[out, in].
"""
from __future__ import annotations

import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight over the last axis; biased variance, no shift."""
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * weight


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / np.sqrt((x ** 2).mean(axis=-1, keepdims=True) + eps) * weight


def rotate_interleaved(x, positions, dims, base):
    """Turns the pairs (2i, 2i+1), i < dims/2, of the last axis of x [T, ..., n] by the angle p * base^(-2i/dims);
    channels from `dims` on pass unchanged."""
    out = np.array(x, dtype=np.float64, copy=True)
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]            # [T, half]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def sink_softmax_mix(scores, sink, values):
    """Rows of `scores` [T, S] (masked entries are -inf) become weights whose denominator also holds exp(sink);
    returns weights @ values."""
    top = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - top)
    denom = e.sum(axis=-1, keepdims=True) + np.exp(sink - top)
    return (e / denom) @ values


def rotation_of(m):
    """(dims, base) of a mixer's rotation; a mixer without rotated channels may leave it out."""
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    return rot["dims"], rot["base"]


def latent_keys(h, m, w, prefix, eps, positions):
    """The latent c [T, kv_rank] and the rotated shared key part [T, rot_dim] of a layer that owns a W_dkv."""
    rank, rot_dim = m["kv_rank"], m["rot_dim"]
    down = h @ w[prefix + "dkv"].T
    c = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, rank:rank + rot_dim], positions, *rotation_of(m))
    return c, k_rot


def latent_attention(h, m, w, prefix, eps, positions, c, k_rot):
    """The mixer's output for the rows h, given the latent and the rotated key part (its own or another layer's)."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim + rot_dim)
    q_plain = q[:, :, :dim]
    q_rot = rotate_interleaved(q[:, :, dim:], positions, *rotation_of(m))
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, dim)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, vdim)
    causal = np.tril(np.ones((T, T), dtype=bool))
    mixed = np.zeros((T, H, vdim))
    for head in range(H):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        scores = np.where(causal, scores, -np.inf)
        mixed[:, head] = sink_softmax_mix(scores, w[prefix + "sink"][head], v[:, head])
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (mixed.reshape(T, H * vdim) * gate) @ w[prefix + "o"].T


def lightning(h, m, w, prefix, eps):
    """Linear attention with a per-head decay, token by token from a zero state."""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[prefix + "q"].T).reshape(T, H, dim)
    k = silu(h @ w[prefix + "k"].T).reshape(T, H, dim)
    v = silu(h @ w[prefix + "v"].T).reshape(T, H, vdim)
    out = np.zeros((T, H, vdim))
    for head in range(H):
        state = np.zeros((dim, vdim))
        for t in range(T):
            state = m["decay"][head] * state + np.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    normed = rms_norm(out.reshape(T, H * vdim), w[prefix + "norm"], eps)
    return (normed * sigmoid(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


def dense_feed_forward(h, w, prefix):
    return (gelu_tanh(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def forward(config, w, tokens, *, return_layers=False):
    """Logits [T, vocab] of one sequence; with `return_layers` also the residual stream after every layer."""
    eps = config["norm"]["eps"]
    positions = np.arange(len(tokens))
    x = w["embed"][np.asarray(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    latents = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        h = layer_norm(x, w[f"l{i}.norm1"], eps)
        prefix = f"l{i}.mix."
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                latents[i] = latent_keys(h, m, w, prefix, eps, positions)
                source = i
            c, k_rot = latents[source]
            x = x + latent_attention(h, m, w, prefix, eps, positions, c, k_rot)
        elif layer["type"] == "lightning":
            x = x + lightning(h, m, w, prefix, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(layer_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp.")
        after.append(x.copy())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T * config.get("logit_scale", 1.0)
    return (logits, np.stack(after)) if return_layers else logits
