"""Norms.  A norm reads rows of the float32 residual stream and writes rows in the activation dtype."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import register_part


@register_part("norm", "layernorm")
class LayerNorm:
    """y = (x − mean)·(1/sqrt(var + eps))·weight + bias over the last axis, biased variance, statistics
    in float32 (reference: include/model/ops.hpp:443-476)."""

    #: what a product kernel may compute in its own prologue instead of calling this norm: a mixer or feed-forward
    #: that is handed the norm looks here (and at weight / bias / eps), never at the class
    fusable_as = "layernorm"

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, eps: float):
        if weight.shape != bias.shape or weight.dim() != 1:
            raise ValueError("LayerNorm: weight and bias are vectors of one length")
        self.weight, self.bias, self.eps = weight, bias, float(eps)
        self.width = weight.shape[0]

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """out[r] = LN(x[rows[r]]) when `rows` is given, else row by row."""
        ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out
