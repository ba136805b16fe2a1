"""A matrix memory with exponential gates: a recurrent state instead of cached keys."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CacheNeed, StateSpec
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear


def _round_up(n: int, to: int) -> int:
    return -(-n // to) * to


class MatrixMemory(Mixer):
    """Per head a matrix S (dim x vdim), a vector n (dim) and a running maximum m (all 32-bit, zero for a new sequence):

        q = W_q h * dim^-1/2,  k = W_k h,  v = W_v h
        a = cap tanh((W_i h + b_i) / cap)                       log of the input gate, one number a head
        b = log sigmoid(cap tanh((W_f h + b_f) / cap))          log of the forget gate
        m_t = max(b_t + m_(t-1), a_t)
        S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T        (n_t likewise, with k_t alone)
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

    Every head's o_t is divided by its own root mean square (eps inside the root); the heads side by side are multiplied
    by a weight and by sigmoid(W_g h) and projected by W_o into the residual stream, times `out_scale`.  Gates, the
    recurrence, the norm and the output gate run in 32-bit (csrc/mlstm.cu, csrc/rowwise.cu).  The state is the layer's
    only cache: `StateSpec`s "s" (heads, dim, vdim), "n" (heads, dim), "m" (heads), one row per live sequence.

    Tensors (stored [out, in]): `in.weight` = rows of W_q, W_k, W_v, W_g, W_i, W_f and zero rows up to a multiple of
    8 (`in_width`); `i.bias`, `f.bias` [heads]; `norm.weight` [heads * vdim]; `out.weight` [width, heads * vdim].
    """

    accepts_lazy_norm = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, gate_cap: float, eps: float, *,
                 out_scale: float = 1.0, init_std: float = 0.02, out_init_std: float | None = None):
        if min(width, n_heads, dim, vdim) <= 0:
            raise ShapeError("matrix memory: sizes must be positive")
        if dim > 256:
            raise ShapeError(f"matrix memory: {dim} key channels per head exceed the 256 the recurrence kernel takes")
        if not gate_cap > 0:
            raise ShapeError(f"matrix memory: the gates' cap must be positive, found {gate_cap}")
        self.width, self.n_heads, self.dim, self.vdim = width, n_heads, dim, vdim
        self.gate_cap, self.eps, self.out_scale = float(gate_cap), float(eps), float(out_scale)
        self.qk_width, self.v_width = n_heads * dim, n_heads * vdim
        self.gates_width = _round_up(2 * n_heads, 8)
        self.in_width = 2 * self.qk_width + 2 * self.v_width + self.gates_width
        # channels of the in-projection's rows
        self.q_off, self.k_off, self.v_off = 0, self.qk_width, 2 * self.qk_width
        self.g_off = self.v_off + self.v_width
        self.i_off = self.g_off + self.v_width
        self.f_off = self.i_off + n_heads
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        return {"in.weight": TensorSpec((self.in_width, self.width), MATRIX, ("normal", self.init_std)),
                "i.bias": TensorSpec((self.n_heads,), VECTOR, ("zeros",)),
                "f.bias": TensorSpec((self.n_heads,), VECTOR, ("zeros",)),
                "norm.weight": TensorSpec((self.v_width,), VECTOR, ("ones",)),
                "out.weight": TensorSpec((self.width, self.v_width), MATRIX, ("normal", self.out_init_std))}

    def bind(self, tensors):
        super().bind(tensors)
        # the output's scale rides on the norm's 32-bit weight
        self.norm_scaled = self.t_norm_weight if self.out_scale == 1.0 else self.t_norm_weight * self.out_scale

    def cache_need(self):
        heads, f32 = self.n_heads, torch.float32
        return CacheNeed(states=(StateSpec("s", (heads, self.dim, self.vdim), f32), StateSpec("n", (heads, self.dim), f32),
                                 StateSpec("m", (heads,), f32)))

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a matrix memory has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("matrix memory: a recurrent state cannot be another layer's")
        mark = ctx.ws.mark()      # (this layer's scratch is handed out again to the next one)
        n = ctx.n_tokens
        proj = ctx.ws.take((n, self.in_width), ctx.dtype)
        linear(ctx, x, self.t_in_weight, None, proj, m=n, w_is_nk=True)
        read = ctx.ws.take((n, self.v_width), torch.float32)
        scratch = None
        if ctx.max_new > kernels.MLSTM_CHUNK:
            # long runs of new tokens: the chunks of a run are worked side by side (csrc/mlstm.cu)
            scratch = ctx.ws.take((kernels.mlstm_chunked_scratch_floats(n, ctx.n_seqs, ctx.max_new, self.n_heads, self.dim,
                                                                        self.vdim),), torch.float32)
        mixed = ctx.ws.take((n, self.v_width), ctx.dtype)
        normed = kernels.mlstm_scan(proj, (self.q_off, self.k_off, self.v_off, self.i_off, self.f_off), self.t_i_bias, self.t_f_bias,
                           self.gate_cap, self.dim ** -0.5, ctx.cache.state(entry, "s"), ctx.cache.state(entry, "n"),
                           ctx.cache.state(entry, "m"), ctx.slots, ctx.seq_start, read, n_seqs=ctx.n_seqs,
                           n_heads=self.n_heads, dim=self.dim, vdim=self.vdim, max_new=ctx.max_new, scratch=scratch,
                                    norm=(self.norm_scaled, self.eps, self.g_off, mixed))
        if not normed:       # (long runs, and heads too large for one block of the token-by-token kernel)
            kernels.rmsnorm(read, self.norm_scaled, mixed, self.eps, n_rows=n, gate=proj[:, self.g_off:self.g_off + self.v_width],
                            groups=self.n_heads)
        linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)
