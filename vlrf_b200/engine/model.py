"""A decoder model as data: parts, layers, and the order in which the layers run.

`DecoderModel` knows no architecture.  An architecture's builder (see `vlrf_b200.models`) makes the
parts from a configuration and the checked weights and hands them over with a *schedule*: the list of
layer calls of one forward pass.  A call names the layer to run, so a layer may appear twice, and may
name an earlier call whose cache it reads instead of keeping one of its own.
"""
from __future__ import annotations

import dataclasses

import torch

from ..parts.context import StepContext


@dataclasses.dataclass(frozen=True)
class LayerCall:
    layer: int                    # index into DecoderModel.layers
    reads_cache_of: int | None = None   # index of an earlier call in the schedule, or None: own cache


@dataclasses.dataclass
class BuildOptions:
    dtype: torch.dtype            # torch.bfloat16 (serving kernels) or torch.float32 (everything 32-bit)
    device: torch.device


class DecoderModel:
    def __init__(self, *, config, embedding, layers, schedule, final_norm, head, options: BuildOptions,
                 max_seq_len: int):
        self.config = config
        self.embedding, self.layers, self.final_norm, self.head = embedding, list(layers), final_norm, head
        self.schedule = [c if isinstance(c, LayerCall) else LayerCall(int(c)) for c in schedule]
        self.options = options
        self.act_dtype = options.dtype
        self.device = options.device
        self.max_seq_len = int(max_seq_len)
        self.width = embedding.width
        self.vocab_size = head.vocab_size
        for i, call in enumerate(self.schedule):
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {call.layer}, which does not exist")
            if call.reads_cache_of is not None:
                j = call.reads_cache_of
                if not (0 <= j < i) or self.schedule[j].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {i} must read the cache of an earlier entry that owns one")
                if self.layers[self.schedule[j].layer].cache_need() != self.layers[call.layer].cache_need():
                    raise ValueError(f"schedule entry {i} reads a cache whose shape differs from its own need")

    @property
    def replayable(self) -> bool:
        """Whether a step's launches may be captured in a CUDA graph and replayed: every part must enqueue the
        same work for the same shapes without asking the device anything.  A part whose control flow
        depends on device values (say, a feed-forward that gathers each expert's tokens on the host) says
        so with a class or instance attribute `replayable = False`; steps then launch plainly."""
        cached = self.__dict__.get("_replayable")          # (asked at every step; the parts of a model do not change)
        if cached is not None:
            return cached

        def ok(obj):
            return getattr(obj, "replayable", True)
        parts = [self.embedding, self.final_norm, self.head]
        for layer in self.layers:
            parts.append(layer)
            parts.extend(v for v in vars(layer).values() if not isinstance(v, (int, float, str, torch.Tensor)))
        self.__dict__["_replayable"] = all(ok(p) for p in parts)
        return self.__dict__["_replayable"]

    def describe_kernels(self, block_tokens: int = 64) -> list:
        """For every layer whose mixer can say, which attention kernels its sizes get (see the mixers' `kernels`)."""
        out = []
        for i, layer in enumerate(self.layers):
            mixer = getattr(layer, "mixer", None)
            if mixer is not None and hasattr(mixer, "kernels"):
                out.append((i, type(mixer).__name__, mixer.kernels(self.act_dtype, block_tokens)))
        return out

    def cache_needs(self) -> list:
        """For every schedule entry what it keeps per sequence (None for entries that read another's)."""
        return [None if c.reads_cache_of is not None else self.layers[c.layer].cache_need()
                for c in self.schedule]

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif hasattr(obj, "__dict__"):
                for v in vars(obj).values():
                    visit(v)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)

        for part in (self.embedding, self.layers, self.final_norm, self.head):
            visit(part)
        return total

    def emit_decode(self, program, cache) -> torch.Tensor:
        """The same forward pass for a decode step (one token a row, logits for every row), written down as the
        operations of a decode program (`parts.program.DecodeProgram`) instead of being launched.  Returns the
        float32 logits tensor [rows, vocab] that running the program fills.  Raises `NotFusable` if a part cannot
        state its step that way; the step then runs through `forward` as always."""
        from ..parts.program import NotFusable
        rows = program.n_rows
        for part in (self.embedding, self.head, *self.layers):
            if not hasattr(part, "emit_decode"):
                raise NotFusable(f"{type(part).__name__} has no emit_decode")
        x = program.scratch("residual", rows, self.width, torch.float32)
        self.embedding.emit_decode(program, x)
        for i, call in enumerate(self.schedule):
            owner = i if call.reads_cache_of is None else call.reads_cache_of
            view = cache.view(owner) if cache.needs[owner] is not None else None
            self.layers[call.layer].emit_decode(program, x, view, writes_cache=call.reads_cache_of is None)
        logits = program.plain("logits", rows, self.vocab_size, torch.float32)
        self.head.emit_decode(program, x, self.final_norm, logits)
        return logits

    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        """Run the tokens of `ctx` through all scheduled layers; returns float32 logits
        [ctx.n_logit_rows, vocab] for the rows in ctx.logit_rows
        (reference: include/model/transformer.hpp:335-424, which keeps the last row only)."""
        x = ctx.ws.get("residual", ctx.n_tokens, self.width, torch.float32)
        ctx.ws.row_stats.forget()                      # nothing is known about the rows of the step before
        self.embedding(ctx, x)
        if not getattr(self.embedding, "leaves_row_stats", False):
            ctx.ws.row_stats.forget()
        for i, call in enumerate(self.schedule):
            owner = i if call.reads_cache_of is None else call.reads_cache_of
            view = cache.view(owner) if cache.needs[owner] is not None else None
            self.layers[call.layer].forward(x, ctx, view, writes_cache=call.reads_cache_of is None)
            if not getattr(self.layers[call.layer], "leaves_row_stats", False):
                ctx.ws.row_stats.forget()              # a block of another kind that does not vouch for them
        n = ctx.n_logit_rows
        logits = ctx.ws.get("logits", max(n, 1), self.vocab_size, torch.float32)
        if n == 0:
            return logits[:0]
        hn = ctx.ws.get("final_normed", n, self.width, ctx.act_dtype)
        self.final_norm(x, hn, ctx.logit_rows)
        self.head(hn, logits, n)
        return logits[:n]
