"""Blocks: how a layer arranges its norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .context import StepContext
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += ffn(norm2(x)) (reference: include/model/transformer_block.hpp:149-159).
    The residual stream x stays float32; the normed rows are in the activation dtype."""

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def leaves_row_stats(self) -> bool:
        """Whether the step's row statistics are true after this block: its last part says (see forward)."""
        return bool(getattr(self.feed_forward, "leaves_row_stats", False))

    def emit_decode(self, program, x: torch.Tensor, view, writes_cache: bool = True) -> None:
        """This block's decode step as operations of a decode program: possible when the mixer and the
        feed-forward can state theirs (they get the norm to fuse, as in `forward`)."""
        from .program import NotFusable
        for part in (self.mixer, self.feed_forward):
            if not hasattr(part, "emit_decode"):
                raise NotFusable(f"{type(part).__name__} has no emit_decode")
        self.mixer.emit_decode(program, x, self.norm1, view, writes_cache)
        self.feed_forward.emit_decode(program, x, self.norm2)

    def forward(self, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True) -> None:
        if getattr(self.mixer, "fuses_norm", False):
            self.mixer.forward(None, x, ctx, view, writes_cache, norm=self.norm1)
        else:
            h = ctx.ws.get("block_normed", ctx.n_tokens, x.shape[1], ctx.act_dtype)
            self.mixer.forward(self.norm1(x, h), x, ctx, view, writes_cache)
        # What is known about the residual rows (their statistics, for a fused LayerNorm) is true only if the part
        # that just rewrote them says so; a part with kernels of its own need not know that such a thing exists.
        if not getattr(self.mixer, "leaves_row_stats", False):
            ctx.ws.row_stats.forget()
        if getattr(self.feed_forward, "fuses_norm", False):
            self.feed_forward.forward(None, x, ctx, norm=self.norm2)
        else:
            h = ctx.ws.get("block_normed", ctx.n_tokens, x.shape[1], ctx.act_dtype)
            self.feed_forward.forward(self.norm2(x, h), x, ctx)
        if not getattr(self.feed_forward, "leaves_row_stats", False):
            ctx.ws.row_stats.forget()
