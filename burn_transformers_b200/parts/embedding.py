"""Token embedding and the readout."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Part
from .linear import linear


class TokenEmbedding(Part):
    """x0[t] = (table[id[t]] (+ the position table's row when the position encoding is a learned one)) * scale,
    the scaling in 32-bit."""

    def __init__(self, vocab: int, width: int, init_std: float = 0.02, scale: float = 1.0):
        self.vocab, self.width, self.init_std, self.scale = vocab, width, init_std, float(scale)

    def specs(self):
        return {"weight": TensorSpec((self.vocab, self.width), MATRIX, ("normal", self.init_std))}

    def forward(self, ctx, positions_part, out32):
        table = positions_part.t_weight if getattr(positions_part, "adds_to_embedding", False) else None
        program = getattr(ctx, "program", None)
        if program is not None:
            if self.scale != 1.0:
                from ..engine.program import ProgramUnsupported
                raise ProgramUnsupported("a scaled embedding has no phase in the fused step")
            program.add_embed(ctx.tokens, ctx.positions if table is not None else None, self.t_weight, table, out32)
            return
        kernels.embed(ctx.tokens, ctx.positions, self.t_weight, table, out32, status=None, scale=self.scale)


class StreamVectors(Part):
    """A table of learned vectors [count, width], one of which is added to every row of the residual stream where the
    model's run order says so (a run of layers that is repeated opens each pass with its own vector).  Kept in 32-bit:
    the sum is part of the stream."""

    def __init__(self, count: int, width: int, init_std: float = 0.02):
        self.count, self.width, self.init_std = count, width, init_std

    def specs(self):
        return {"weight": TensorSpec((self.count, self.width), VECTOR, ("normal", self.init_std))}

    def forward(self, ctx, residual, index: int):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a vector added between layers has no phase in the fused step")
        if not 0 <= index < self.count:
            raise IndexError(f"vector {index} of {self.count}")
        kernels.add_vector(residual, self.t_weight[index], n_rows=ctx.n_tokens)


class TiedReadout(Part):
    """logits = h @ table^T with the token embedding's table, no bias, 32-bit logits
    (src/models/gpt2/model.rs:496-513).  Owns no tensor: it borrows the embedding's."""

    accepts_lazy_norm = True

    def __init__(self, embedding: TokenEmbedding):
        self.embedding = embedding

    def forward(self, ctx, h, n_rows: int):
        logits = ctx.ws.take((n_rows, self.embedding.vocab), torch.float32)
        linear(ctx, h, self.embedding.t_weight, None, logits, m=n_rows, w_is_nk=True)
        return logits


class LinearReadout(Part):
    """logits = (h @ weight^T) * scale with a table of its own, stored [vocab, width]; no bias, 32-bit logits, the
    scaling in 32-bit."""

    accepts_lazy_norm = True

    def __init__(self, vocab: int, width: int, scale: float = 1.0, init_std: float = 0.02):
        self.vocab, self.width, self.scale, self.init_std = vocab, width, float(scale), init_std

    def specs(self):
        return {"weight": TensorSpec((self.vocab, self.width), MATRIX, ("normal", self.init_std))}

    def forward(self, ctx, h, n_rows: int):
        logits = ctx.ws.take((n_rows, self.vocab), torch.float32)
        linear(ctx, h, self.t_weight, None, logits, m=n_rows, w_is_nk=True)
        if self.scale != 1.0:
            if getattr(ctx, "program", None) is not None:
                from ..engine.program import ProgramUnsupported
                raise ProgramUnsupported("a scaled readout has no phase in the fused step")
            kernels.scale_(logits, self.scale)
        return logits
