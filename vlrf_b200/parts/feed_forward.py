"""Feed-forward parts.

Interface: forward(h, x, ctx): x += ffn(h) in place; h is the normed input [n_tokens, width] in the
activation dtype, x the float32 residual stream.  A part with routing and experts would have the same
interface and own its router.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext
from .registry import register_part

ACTIVATIONS = ("gelu_tanh", "gelu_erf")


@register_part("feed_forward", "dense_mlp")
class DenseMLP:
    """x += act(h·W_inᵀ + b_in)·W_outᵀ + b_out; the activation runs in the first product's epilogue and
    the residual sum in the second's (reference: include/model/feedforward.hpp:50-77,
    include/model/transformer_block.hpp:158; tanh GELU include/model/ops.hpp:390-403)."""

    def __init__(self, w_in, b_in, w_out, b_out, *, activation: str):
        if activation not in ACTIVATIONS:
            raise ValueError(f"DenseMLP: activation '{activation}' is not one of {', '.join(ACTIVATIONS)}")
        if w_out.shape[1] != w_in.shape[0] or w_out.shape[0] != w_in.shape[1]:
            raise ValueError("DenseMLP: the two matrices do not chain")
        self.w_in, self.b_in, self.w_out, self.b_out = w_in, b_in, w_out, b_out
        self.activation = activation
        self.inner = w_in.shape[0]

    #: the block may hand over its norm instead of normed rows: forward(None, x, ctx, norm=…)
    fuses_norm = True
    #: the residual rows are written last by a product that is handed the step's row statistics (see the mixer)
    leaves_row_stats = True

    def emit_decode(self, program, x: torch.Tensor, norm) -> None:
        """The decode step of this part as two operations of a decode program."""
        from .program import norm_terms
        u = program.scratch("ffn_inner", program.n_rows, self.inner, program.act_dtype)
        program.product(x, self.w_in, self.b_in, u, norm=norm_terms(norm), act=self.activation)
        program.product(u, self.w_out, self.b_out, x, residual=x)

    def forward(self, h, x: torch.Tensor, ctx: StepContext, norm=None) -> None:
        T = ctx.n_tokens
        u = ctx.ws.get("ffn_inner", T, self.inner, ctx.act_dtype)
        if h is None and getattr(norm, "fusable_as", None) == "layernorm" and ops.can_fuse_layernorm(T, x.shape[1], self.w_in.dtype):
            ops.linear_layernorm(x, norm.weight, norm.bias, norm.eps, self.w_in, self.b_in, u, act=self.activation,
                                 stats=ctx.ws.row_stats)
        else:
            if h is None:
                h = norm(x, ctx.ws.get("block_normed", T, x.shape[1], ctx.act_dtype))
            ops.linear(h, self.w_in, self.b_in, u, act=self.activation)
        ops.linear(u, self.w_out, self.b_out, x, residual=x, stats=ctx.ws.row_stats)
