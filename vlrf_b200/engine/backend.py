"""The generation loop's backend on the device: `Engine.step` for steps that bring prompts, a `DecodeSession` for
the steps in which every row goes on by one token, and the sampling kernels.

A table of rows holds sequences in turn.  The decode session spans the whole table (rows that hold nothing are
padding), so its captured step stays valid while requests come and go: a row that is taken or given back changes
entries of the session's device tables, not their addresses.  A step that brings a prompt (a request was just
admitted) runs through `Engine.step`, prompts and single tokens in one flat batch; the session's tables are brought
up to date before its next step."""
from __future__ import annotations

import dataclasses

import torch

from ..sampling.params import SamplingParams
from ..sampling.rng import request_key
from ..sampling.sampler import RowSampler
from .decode import DecodeSession
from .step import Engine, StepEntry


@dataclasses.dataclass
class _Table:
    slots: list                       # the cache slot of every row, or None
    sampler: RowSampler
    most_tokens: list                 # most tokens each row's sequence may come to hold
    session: DecodeSession | None = None
    stale: bool = True                # the session's device tables lag behind the cache's books
    staging: torch.Tensor | None = None   # pinned host int32: the tokens fed at a decode step
    result: torch.Tensor | None = None    # pinned host int32: the tokens a decode step chose
    staging_np: object = None             # numpy view of `staging`
    graph_calls: tuple | None = None      # (feed, choose, fetch) of the replayed step, made once
    stream: object = None                 # the stream the table's steps run on (the current one when decoding began)


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class DeviceBackend:
    def __init__(self, engine: Engine, *, use_graph: bool = True):
        self.engine = engine
        self.use_graph = use_graph
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.decode_steps = 0
        self.prompt_steps = 0

    def limits(self):
        c = self.engine.cache
        return c.max_tokens, c.n_slots, c.block_tokens, self.engine.model.max_seq_len

    def open_table(self, n_rows: int, requests: list) -> _Table:
        """`requests`: every request that may ever be admitted to the table; what any of them needs (a random draw,
        penalties, a history of so many tokens) the table's sampler is set up for, once."""
        history = max((r.params.max_new_tokens for r in requests), default=1)
        greedy = SamplingParams(do_sample=False)
        sampler = RowSampler([greedy] * n_rows, [0] * n_rows, self.engine.device, history,
                             any_sampling=any(not r.params.greedy for r in requests),
                             any_penalties=any(r.params.has_penalties for r in requests))
        return _Table([None] * n_rows, sampler, [0] * n_rows)

    def admit(self, table: _Table, row: int, request) -> None:
        if table.slots[row] is not None:
            raise ValueError(f"row {row} still holds a sequence")
        slot = self.engine.start_sequence()
        table.slots[row] = slot
        table.most_tokens[row] = min(len(request.prompt) + max(request.params.max_new_tokens - 1, 0),
                                     self.engine.model.max_seq_len)
        table.sampler.set_row(row, request.params, request_key(request.params.seed, request.index))
        if table.session is not None:
            table.session.take_row(row, slot)
        table.stale = True

    def run(self, table: _Table, rows: list, tokens: list) -> list:
        decode = all(len(t) == 1 for t in tokens) and all(self.engine.length(table.slots[r]) > 0 for r in rows)
        if decode:
            if table.session is None:
                # every live row goes on by one token: from here on such steps are replayed
                n = len(table.slots)
                table.session = DecodeSession(self.engine, list(table.slots), use_graph=self.use_graph, pad_to=_bucket(n))
                table.staging = torch.zeros(n, dtype=torch.int32, pin_memory=True)
                table.result = torch.zeros(n, dtype=torch.int32, pin_memory=True)
                table.staging_np = table.staging.numpy()
                table.stream = torch.cuda.current_stream()
                table.stale = True
            if table.stale:
                # blocks for all that the rows' sequences may come to hold, so that replayed steps need no change of the
                # block tables; then slot and position of every row as the cache's books have them
                for slot, most in zip(table.slots, table.most_tokens):
                    if slot is not None:
                        self.engine.cache.reserve(slot, most)
                self.engine.cache.sync_tables()
                table.session.sync_tables()
                table.stale = False
            return self._run_decode(table, rows, tokens)
        entries = [StepEntry(table.slots[r], toks, [len(toks) - 1]) for r, toks in zip(rows, tokens)]
        logits = self.engine.step(entries)
        out = table.sampler.sample(logits, rows)
        host = out.tolist()                      # the step's one device→host read; synchronises
        table.stale = True                       # positions moved on without the session
        self.prompt_steps += 1
        self.h2d_bytes += 4 * (3 * sum(len(t) for t in tokens) + 4 * len(rows) + 1)
        self.d2h_bytes += 4 * len(rows)
        self.engine.check_device_errors()
        return host

    def _run_decode(self, table: _Table, rows: list, tokens: list) -> list:
        sess = table.session
        n = len(table.slots)
        st = table.staging_np                                  # (a view of the pinned buffer)
        for r, toks in zip(rows, tokens):
            st[r] = toks[0]
        sampler = table.sampler
        if not sampler.any_penalties:
            # One replayed graph a step: this step's inputs host → device, the model, the sampling kernel
            # (which also moves the positions on), the result device → host.
            if table.graph_calls is None:
                # (the three name the tensors, not the table: a table that held functions that hold the table would
                # be cyclic garbage, and its graph would wait for a collection at some later, arbitrary moment)
                staging, result = table.staging, table.result
                everyone = list(range(n))

                def feed():
                    sess.tokens[:n].copy_(staging, non_blocking=True)

                def choose(logits):
                    sampler.sample(logits[:n], everyone, next_pos=sess.tok_pos, row_slot=sess.tok_slot)

                def fetch():
                    result.copy_(sampler.out[:n], non_blocking=True)

                table.graph_calls = (feed, choose, fetch)
            feed, choose, fetch = table.graph_calls
            sess.step_sampled(choose, key=sampler, state=(sampler.rng_ctr,), before=feed, after=fetch)
            table.stream.synchronize()                         # the step's result is in host memory
            host = table.result.tolist()
        else:
            sess.tokens[:n].copy_(table.staging, non_blocking=True)    # this step's inputs, host → device
            logits = sess.step(advance_on_device=False)            # the sampling kernel moves the positions on
            out = sampler.sample(logits[:n], list(range(n)), next_pos=sess.tok_pos, row_slot=sess.tok_slot)
            host = out.tolist()                                    # this step's result, device → host; synchronises
        self.h2d_bytes += 4 * n
        self.d2h_bytes += 4 * n
        self.decode_steps += 1
        return [host[r] for r in rows]

    def close_row(self, table: _Table, row: int) -> None:
        slot = table.slots[row]
        if slot is None:
            raise ValueError(f"row {row} holds no sequence")
        if table.session is not None:
            table.session.end_row(row)
        self.engine.end_sequence(slot)
        table.slots[row] = None

    def close_table(self, table: _Table) -> None:
        for row, slot in enumerate(table.slots):
            if slot is not None:
                self.close_row(table, row)
        table.session = None
        table.graph_calls = None
