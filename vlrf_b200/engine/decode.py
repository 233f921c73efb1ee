"""Decoding a fixed set of sequences one token per step, with the tokens staying on the device.

A `DecodeSession` is the step function specialised to "every sequence goes on by one token": the
integer tables of the step (token, slot, position per row) are static device tensors, so the step's
launches can be captured once in a CUDA graph and replayed, and the sampled tokens of one step are
written straight into the token table of the next.  It runs the same `DecoderModel.forward` on the same
cache as `Engine.step`; rows of ended sequences become padding (slot −1), which every part skips.
"""
from __future__ import annotations

import torch

import os

from ..csrc import launch_count
from .capture import capture_into
from ..parts.context import StepContext, Workspace
from .step import Engine


#: Whether a session states its step as a decode program (one persistent kernel a step) where the model's parts
#: allow it; off, or for models whose parts cannot, every operation is a launch of its own.
USE_DECODE_PROGRAM = os.environ.get("VLRF_B200_DECODE_PROGRAM", "0") != "0"


class DecodeSession:
    def __init__(self, engine: Engine, slots: list, *, use_graph: bool = True, pad_to: int | None = None,
                 use_program: bool | None = None):
        self.engine, self.model = engine, engine.model
        self.slots = list(slots)         # a row's cache slot, or None for a row that holds no sequence (yet)
        self.n = len(slots)
        self.rows = pad_to if pad_to is not None else self.n
        if self.rows < self.n:
            raise ValueError("pad_to is smaller than the number of sequences")
        dev = engine.device
        self.live = [s is not None for s in self.slots]
        self.tokens = torch.zeros(self.rows, dtype=torch.int32, device=dev)
        self.tok_slot = torch.full((self.rows,), -1, dtype=torch.int32, device=dev)
        self.tok_pos = torch.zeros(self.rows, dtype=torch.int32, device=dev)
        self.seq_start = torch.arange(self.rows + 1, dtype=torch.int32, device=dev)
        self.logit_rows = torch.arange(self.rows, dtype=torch.int32, device=dev)
        self.one = torch.ones(self.rows, dtype=torch.int32, device=dev)
        self.ws = Workspace(dev)
        self.use_graph = use_graph and self.model.replayable
        self.graph = None
        self._greedy_graph = None
        self._greedy_out = None
        self.logits = None
        self.kernels_per_step = 0
        self._sync_tables()
        self.program = None
        self.program_refused = None      # why the step is not a decode program, if it is not
        if USE_DECODE_PROGRAM if use_program is None else use_program:
            self._build_program()

    def _build_program(self) -> None:
        from ..parts.program import DecodeProgram, NotFusable
        try:
            if not self.model.replayable:
                raise NotFusable("a part of the model decides on the host what to launch")
            program = DecodeProgram(n_rows=self.rows, tokens=self.tokens, tok_slot=self.tok_slot, tok_pos=self.tok_pos,
                                    dev_err=self.engine.dev_err, ws=self.ws, act_dtype=self.model.act_dtype,
                                    max_context=self.model.max_seq_len)
            self._program_logits = self.model.emit_decode(program, self.engine.cache)
            program.finalize()
            self.program = program
        except NotFusable as why:
            self.program_refused = str(why)

    def _run_model(self) -> torch.Tensor:
        """The model on this step's rows: one launch of the decode program where there is one."""
        if self.program is not None:
            self.program.run()
            return self._program_logits
        return self.model.forward(self._context(), self.engine.cache)

    def _sync_tables(self) -> None:
        c = self.engine.cache
        slot = [s if live else -1 for s, live in zip(self.slots, self.live)] + [-1] * (self.rows - self.n)
        pos = [c.lengths[s] if live else 0 for s, live in zip(self.slots, self.live)] + [0] * (self.rows - self.n)
        self.tok_slot.copy_(torch.tensor(slot, dtype=torch.int32), non_blocking=False)
        self.tok_pos.copy_(torch.tensor(pos, dtype=torch.int32), non_blocking=False)

    def set_tokens(self, tokens) -> None:
        """The tokens to feed at the next step: a device int32 tensor [n] or a host list."""
        if isinstance(tokens, torch.Tensor):
            self.tokens[:self.n].copy_(tokens[:self.n])
        else:
            self.tokens[:self.n].copy_(torch.tensor(list(tokens), dtype=torch.int32))

    def step_greedy(self, out: torch.Tensor) -> torch.Tensor:
        """A whole greedy decode step on the device: the model, the argmax, and the hand-over of token and
        position to the next step, captured together; `out` (int32 [rows]) receives the tokens."""
        from ..csrc import ops

        def argmax(logits):
            ops.sample(logits, self.rows, out, next_tokens=self.tokens, next_pos=self.tok_pos, row_slot=self.tok_slot)

        return self.step_sampled(argmax, key=out)

    def step_sampled(self, sample, *, key, state=(), before=None, after=None) -> torch.Tensor:
        """A whole decode step captured as one graph: `before()` (say, a copy of the step's tokens from
        pinned host memory), the model, `sample(logits)` — which must launch the sampling kernel with
        `next_pos=self.tok_pos, row_slot=self.tok_slot` so that the positions move on — and `after()`
        (say, a copy of the result to pinned host memory).  All of them may only enqueue work on tensors
        that stay where they are.  The graph is kept as long as `key` is the same object; `state`:
        tensors that `sample` changes in place (random counters), put back after the uncaptured run that
        sizes the workspace."""
        c = self.engine.cache
        for s, live in zip(self.slots, self.live):
            if live and c.lengths[s] + 1 > self.model.max_seq_len:
                raise ValueError(f"slot {s} is at the model's last position")

        def run():
            if before is not None:
                before()
            logits = self._run_model()
            sample(logits)
            if after is not None:
                after()
            return logits

        if not self.use_graph:
            start = launch_count()
            self.logits = run()
            self.kernels_per_step = launch_count() - start
        else:
            if self._greedy_graph is None or self._greedy_out is not key:
                kept = [t.clone() for t in (self.tok_pos, self.tokens, *state)]   # the warm-up run must not advance anything
                start = launch_count()
                self.logits = run()
                self.kernels_per_step = launch_count() - start
                torch.cuda.synchronize()
                for t, k in zip((self.tok_pos, self.tokens, *state), kept):
                    t.copy_(k)
                self.ws.frozen = True
                g = torch.cuda.CUDAGraph()
                with capture_into(g):
                    self.logits = run()
                self._greedy_graph, self._greedy_out = g, key
            self._greedy_graph.replay()
        for s, live in zip(self.slots, self.live):
            if live:
                c.advance(s, 1)
        self.engine.steps_run += 1
        return self.logits

    def take_row(self, row: int, slot: int) -> None:
        """A free row takes the sequence in `slot` (which already holds its prompt); `sync_tables()` must follow
        before the next step."""
        if self.live[row]:
            raise ValueError(f"row {row} still holds a sequence")
        self.slots[row], self.live[row] = slot, True

    def sync_tables(self) -> None:
        """Bring the device's row tables (slot and position of every row) up to the cache's books: after rows were
        taken, or after steps that ran outside the session."""
        self._sync_tables()

    def end_row(self, row: int) -> None:
        """The sequence of this row has ended; its row becomes padding.  (The slot is the caller's to free.)"""
        self.live[row] = False
        self.tok_slot[row] = -1
        self.tok_pos[row] = 0            # a padding row must not look like a position beyond the table
        self.tokens[row] = 0

    def reserve_ahead(self, n_steps: int) -> None:
        """Make sure every live sequence has blocks for its next n_steps tokens, so that the replayed
        steps need no change of the block tables."""
        c = self.engine.cache
        for s, live in zip(self.slots, self.live):
            if live:
                c.reserve(s, min(c.lengths[s] + n_steps, self.model.max_seq_len))
        c.sync_tables()

    def _context(self) -> StepContext:
        c = self.engine.cache
        most = max([c.lengths[s] + 1 for s, live in zip(self.slots, self.live) if live] or [1])
        return StepContext(
            n_tokens=self.rows, tokens=self.tokens, tok_slot=self.tok_slot, tok_pos=self.tok_pos, n_seqs=self.rows,
            seq_slot=self.tok_slot, seq_start=self.seq_start, seq_pos0=self.tok_pos, max_new=1,
            max_context=self.model.max_seq_len if self.use_graph else most, logit_rows=self.logit_rows,
            n_logit_rows=self.rows, act_dtype=self.model.act_dtype, dev_err=self.engine.dev_err, ws=self.ws,
            host_seq_slots=[s if live else -1 for s, live in zip(self.slots, self.live)], host_seq_lens=[1] * self.rows,
            host_seq_pos0=[])

    def step(self, advance_on_device: bool = True) -> torch.Tensor:
        """One decode step of all rows from `self.tokens`; returns float32 logits [rows, vocab] (static
        storage).  Afterwards every live row's position has advanced by one in the cache's books, and on
        the device too unless `advance_on_device` is False — then whoever samples must pass
        `next_pos=self.tok_pos, row_slot=self.tok_slot` (and `next_tokens=self.tokens`) to the sampling
        kernel, which does it in the same launch."""
        c = self.engine.cache
        for s, live in zip(self.slots, self.live):
            if live and c.lengths[s] + 1 > self.model.max_seq_len:
                raise ValueError(f"slot {s} is at the model's last position")
        if self.use_graph and self.graph is None:
            # a warm-up run sizes the workspace; the capture then sees stable addresses
            before = launch_count()
            self.logits = self._run_model()
            self.kernels_per_step = launch_count() - before
            torch.cuda.synchronize()
            self.ws.frozen = True
            g = torch.cuda.CUDAGraph()
            with capture_into(g):
                self.logits = self._run_model()
            self.graph = g
        if self.use_graph:
            self.graph.replay()
        else:
            before = launch_count()
            self.logits = self._run_model()
            self.kernels_per_step = launch_count() - before
        if advance_on_device:
            self.tok_pos.add_(self.one * (self.tok_slot >= 0))
        for s, live in zip(self.slots, self.live):
            if live:
                c.advance(s, 1)
        self.engine.steps_run += 1
        return self.logits
