"""Token embedding and the head that turns the last hidden rows into logits."""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext


class TokenEmbedding:
    """x[t] = weight[token[t]], fused with a position encoding that acts at the embedding
    (reference: include/model/ops.hpp:615-626, include/model/transformer.hpp:340)."""

    def __init__(self, weight: torch.Tensor, position=None):
        self.weight = weight
        self.vocab_size, self.width = weight.shape
        if position is not None and getattr(position, "where", None) == "embedding":
            if position.table.shape[1] != self.width or position.table.dtype != weight.dtype:
                raise ValueError("TokenEmbedding: the position table does not match the embedding")
            self.position = position
        else:
            self.position = None

    #: the rows are written by a kernel that is handed the step's row statistics (see parts/block.py)
    leaves_row_stats = True

    def emit_decode(self, program, x: torch.Tensor) -> None:
        program.embed(self.weight, self.position.table if self.position is not None else None, x)

    def __call__(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        table = self.position.table if self.position is not None else None
        ops.embed(self.weight, table, ctx.tokens, ctx.tok_pos if table is not None else None, x, ctx.dev_err,
                  stats=ctx.ws.row_stats)
        return x


class LMHead:
    """logits = h · weightᵀ, float32, no bias; a tied head is given the embedding's weight
    (reference: include/model/transformer.hpp:413-414, :298-300)."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.vocab_size, self.width = weight.shape

    def emit_decode(self, program, x: torch.Tensor, norm, logits: torch.Tensor) -> None:
        """logits = norm(x) · weightᵀ for every row of the program."""
        from .program import norm_terms
        program.product(x, self.weight, None, logits, norm=norm_terms(norm))

    def __call__(self, h: torch.Tensor, logits: torch.Tensor, n_rows: int) -> torch.Tensor:
        ops.linear(h, self.weight, None, logits, rows=n_rows)
        return logits
