"""Mixers: the parts that let a token see other tokens.  Attention is the one this library ships.

Interface of a mixer (what `Block` and the step rely on):

    cache_need() -> KVNeed | StateNeed | None     what it keeps per sequence
    forward(h, x, ctx, view, writes_cache=True)   x += mix(h), in place.
        (a mixer that sets `fuses_norm = True` also accepts h=None with `norm=` the block's norm, and
        applies the norm itself, fused where its kernels allow)
        h     [n_tokens, width]  normed input in the activation dtype
        x     [n_tokens, width]  float32 residual stream
        ctx   StepContext        tokens' slots and positions, scratch, error word
        view  CacheView | None   this layer's storage (another layer's when the layer list says so;
                                 then writes_cache is False and the mixer only reads it)
"""
from __future__ import annotations

import torch

from ..cache import KVNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "causal_self_attention")
class CausalSelfAttention:
    """Multi-head causal attention with a fused q/k/v projection over a paged cache.

    q, k, v = h·W_qkvᵀ + b (reference: include/model/attention.hpp:98-105, as one product); k and v
    are written into the cache first (attention.hpp:127-129); every query attends the keys 0…its
    position of its own sequence with score·scale, softmax in float32 (attention.hpp:207-309,
    :373-374); the heads are merged and projected, and the residual is added in the projection's
    epilogue (attention.hpp:183-184, include/model/transformer_block.hpp:153).

    n_kv_heads < n_heads shares each key/value head among n_heads/n_kv_heads query heads; window > 0
    limits a query to the last `window` keys.  GPT-2 uses neither.
    """

    def __init__(self, w_qkv, b_qkv, w_out, b_out, *, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, window: int = 0, position=None):
        width_q, width_kv = n_heads * head_dim, n_kv_heads * head_dim
        if w_qkv.shape[0] != width_q + 2 * width_kv:
            raise ValueError(f"attention: fused projection has {w_qkv.shape[0]} rows, "
                             f"{width_q + 2 * width_kv} expected")
        if w_out.shape[1] != width_q:
            raise ValueError("attention: output projection does not take the merged heads")
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"attention: {n_heads} heads cannot share {n_kv_heads} key/value heads")
        if head_dim % ops.HEAD_DIM_STEP != 0 or not (0 < head_dim <= ops.HEAD_DIM_MAX):
            raise ValueError(f"attention: a head size of {head_dim} is not taken: the attention kernels take head sizes "
                             f"that are multiples of {ops.HEAD_DIM_STEP} up to {ops.HEAD_DIM_MAX}")
        if position is not None and getattr(position, "where", None) == "qk":
            raise NotImplementedError("attention: no position encoding acting on q/k is built into this mixer")
        self.w_qkv, self.b_qkv, self.w_out, self.b_out = w_qkv, b_qkv, w_out, b_out
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.scale, self.window = float(scale), int(window)
        self.q_off, self.k_off, self.v_off = 0, width_q, width_q + width_kv
        self.qkv_width = width_q + 2 * width_kv

    def cache_need(self):
        if self.window > 0:
            return KVNeed(self.n_kv_heads, self.head_dim, "window", self.window)
        return KVNeed(self.n_kv_heads, self.head_dim, "full")

    #: the block may hand over its norm instead of normed rows: forward(None, x, …, norm=…)
    fuses_norm = True
    #: the residual rows are written last by a product of csrc.ops that is handed the step's row statistics, so
    #: what those say afterwards is true (the block forgets them after parts that do not declare this)
    leaves_row_stats = True

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, norm=None) -> None:
        T = ctx.n_tokens
        qkv = ctx.ws.get("attn_qkv", T, self.qkv_width, ctx.act_dtype)
        appended = False
        if h is None and getattr(norm, "fusable_as", None) == "layernorm" and ops.can_fuse_layernorm(T, x.shape[1], self.w_qkv.dtype):
            # few rows: norm, projection and the cache write in one kernel
            scatter = None
            if writes_cache:
                scatter = (view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos, self.k_off, self.v_off,
                           self.n_kv_heads, self.head_dim)
                appended = True
            ops.linear_layernorm(x, norm.weight, norm.bias, norm.eps, self.w_qkv, self.b_qkv, qkv, kv_scatter=scatter,
                                 stats=ctx.ws.row_stats)
        else:
            if h is None:
                h = norm(x, ctx.ws.get("block_normed", T, x.shape[1], ctx.act_dtype))
            scatter = None
            if writes_cache:
                scatter = (view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos, self.k_off, self.v_off,
                           self.n_kv_heads, self.head_dim)
            appended = ops.linear(h, self.w_qkv, self.b_qkv, qkv, kv_scatter=scatter)   # the epilogue writes the cache if it can
        if writes_cache and not appended:
            ops.kv_append(qkv, self.k_off, self.v_off, view.k, view.v, view.block_table, ctx.tok_slot,
                          ctx.tok_pos, T, self.n_kv_heads, self.head_dim, ctx.dev_err)
        merged = ctx.ws.get("attn_out", T, self.n_heads * self.head_dim, ctx.act_dtype)
        self._attend(qkv, view, merged, ctx)
        ops.linear(merged, self.w_out, self.b_out, x, residual=x, stats=ctx.ws.row_stats)

    def emit_decode(self, program, x: torch.Tensor, norm, view, writes_cache: bool = True) -> None:
        """The decode step of this mixer as operations of a decode program: norm + q/k/v projection (+ cache
        write), attention over the cache, output projection + residual."""
        from .program import norm_terms
        rows = program.n_rows
        qkv = program.scratch("attn_qkv", rows, self.qkv_width, program.act_dtype)
        merged = program.scratch("attn_out", rows, self.n_heads * self.head_dim, program.act_dtype, seg=self.head_dim)
        scatter = (view.k, view.v, view.block_table, self.k_off, self.v_off, self.n_kv_heads, self.head_dim) \
            if writes_cache else None
        program.product(x, self.w_qkv, self.b_qkv, qkv, norm=norm_terms(norm), kv_scatter=scatter)
        program.attention(qkv, self.q_off, self.k_off, self.v_off, view.k, view.v, view.block_table, merged, n_heads=self.n_heads,
                          n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, scale=self.scale, window=self.window)
        program.product(merged, self.w_out, self.b_out, x, residual=x)

    def kernels(self, act_dtype: torch.dtype, block_tokens: int) -> dict:
        """Which attention kernels these sizes get: {"prompt": …, "decode": …}, each "tcgen05", "mma.sync" or
        "CUDA cores".  Said once when a model is built, so that a head size that leaves the tensor cores is a
        visible fact."""
        return {"prompt": ops.attention_prefill_kind(act_dtype, self.head_dim, block_tokens, self.qkv_width, self.q_off,
                                                     self.n_heads * self.head_dim),
                "decode": ops.attention_decode_kind(act_dtype, self.head_dim)}

    def _attend(self, qkv, view, merged, ctx: StepContext) -> None:
        T = ctx.n_tokens
        if ctx.max_new == 1:
            # a decode step: few queries, long contexts → split every context across CTAs
            n_split = ops.decode_splits(T, self.n_heads, ctx.max_context)
            partials = counters = None
            if n_split > 1 and ops.attention_decode_needs_scratch(self.head_dim, n_split):
                partials = ctx.ws.get("attn_partials", T * self.n_heads * n_split, self.head_dim + 2, torch.float32)
                counters = ctx.ws.get_zeroed("attn_counters", T * self.n_heads, torch.int32)
            ops.attention_decode(qkv, self.q_off, view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos,
                                 merged, T, self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.window,
                                 n_split, partials, counters, ctx.dev_err)
            return
        if ops.attention_prefill_takes(qkv.dtype, self.head_dim, view.k.shape[2], qkv.shape[1], self.q_off):
            # a prompt step in bfloat16: tiles of 64 queries on the tensor cores
            n_parts = ops.attention_prefill_parts(qkv.dtype, ctx.n_seqs, ctx.max_new, self.n_heads, self.head_dim,
                                                  view.k.shape[2], qkv.shape[1], self.q_off)
            partials = counters = None
            if n_parts > 1:
                n_floats, n_counters = ops.attention_prefill_scratch(ctx.n_seqs, ctx.max_new, self.n_heads, n_parts)
                partials = ctx.ws.get("attn_partials", n_floats, 1, torch.float32)
                counters = ctx.ws.get_zeroed("attn_counters", n_counters, torch.int32)
            ops.attention_prefill(qkv, self.q_off, view.k, view.v, view.block_table, ctx.seq_slot, ctx.seq_start,
                                  ctx.seq_pos0, merged, T, ctx.n_seqs, ctx.max_new, self.n_heads, self.n_kv_heads,
                                  self.head_dim, self.scale, self.window, ctx.dev_err, n_parts, partials, counters)
            return
        ops.attention_generic(qkv, self.q_off, view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos,
                              merged, T, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                              self.window, ctx.dev_err)
