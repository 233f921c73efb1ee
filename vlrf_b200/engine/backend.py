"""The generation loop's backend on the device: `Engine.step` for the prompts, a `DecodeSession` for
the single-token steps, and the sampling kernels."""
from __future__ import annotations

import dataclasses

import torch

from ..sampling.rng import request_key
from ..sampling.sampler import RowSampler
from .decode import DecodeSession
from .step import Engine, StepEntry


@dataclasses.dataclass
class _Batch:
    slots: list
    sampler: RowSampler
    most_tokens: list                 # most tokens each sequence may come to hold
    session: DecodeSession | None = None
    staging: torch.Tensor | None = None   # pinned host int32: the tokens fed at a decode step
    result: torch.Tensor | None = None    # pinned host int32: the tokens a decode step chose
    staging_np: object = None             # numpy view of `staging`
    graph_calls: tuple | None = None      # (feed, choose, fetch) of the replayed step, made once
    stream: object = None                 # the stream the batch's steps run on (the current one when decoding began)


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

    def limits(self):
        c = self.engine.cache
        return c.max_tokens, c.n_slots, c.block_tokens, self.engine.model.max_seq_len

    def open_batch(self, requests: list) -> _Batch:
        slots = [self.engine.start_sequence() for _ in requests]
        keys = [request_key(r.params.seed, r.index) for r in requests]
        history = max((r.params.max_new_tokens for r in requests), default=1)
        sampler = RowSampler([r.params for r in requests], keys, self.engine.device, history)
        most = [min(len(r.prompt) + max(r.params.max_new_tokens - 1, 0), self.engine.model.max_seq_len)
                for r in requests]
        return _Batch(slots, sampler, most)

    def run(self, batch: _Batch, rows: list, tokens: list) -> list:
        if batch.session is None and all(len(t) == 1 for t in tokens) and rows == list(range(len(batch.slots))) \
                and all(self.engine.length(s) > 0 for s in batch.slots):
            # every sequence of the batch goes on by one token: from here on the steps are replayed
            batch.session = DecodeSession(self.engine, batch.slots, use_graph=self.use_graph,
                                          pad_to=_bucket(len(batch.slots)))
            for s, most in zip(batch.slots, batch.most_tokens):
                self.engine.cache.reserve(s, most)
            self.engine.cache.sync_tables()
            batch.staging = torch.zeros(len(batch.slots), dtype=torch.int32, pin_memory=True)
            batch.result = torch.zeros(len(batch.slots), dtype=torch.int32, pin_memory=True)
            batch.staging_np = batch.staging.numpy()
            batch.stream = torch.cuda.current_stream()
        if batch.session is not None:
            return self._run_decode(batch, rows, tokens)
        entries = [StepEntry(batch.slots[r], toks, [len(toks) - 1]) for r, toks in zip(rows, tokens)]
        logits = self.engine.step(entries)
        out = batch.sampler.sample(logits, rows)
        host = out.tolist()                      # the step's one device→host read; synchronises
        self.h2d_bytes += 4 * (3 * sum(len(t) for t in tokens) + 4 * len(rows) + 1)
        self.d2h_bytes += 4 * len(rows)
        self.engine.check_device_errors()
        return host

    def _run_decode(self, batch: _Batch, rows: list, tokens: list) -> list:
        sess = batch.session
        n = len(batch.slots)
        st = batch.staging_np                                  # (a view of the pinned buffer)
        for r, toks in zip(rows, tokens):
            st[r] = toks[0]
        sampler = batch.sampler
        if not sampler.any_penalties:
            # One replayed graph a step: this step's inputs host → device, the model, the sampling kernel
            # (which also moves the positions on), the result device → host.
            if batch.graph_calls is None:
                # (the three name the tensors, not the batch: a batch that held functions that hold the batch would
                # be cyclic garbage, and its graph would wait for a collection at some later, arbitrary moment)
                staging, result = batch.staging, batch.result
                everyone = list(range(n))

                def feed():
                    sess.tokens[:n].copy_(staging, non_blocking=True)

                def choose(logits):
                    sampler.sample(logits[:n], everyone, next_pos=sess.tok_pos, row_slot=sess.tok_slot)

                def fetch():
                    result.copy_(sampler.out[:n], non_blocking=True)

                batch.graph_calls = (feed, choose, fetch)
            feed, choose, fetch = batch.graph_calls
            sess.step_sampled(choose, key=sampler, state=(sampler.rng_ctr,), before=feed, after=fetch)
            batch.stream.synchronize()                         # the step's result is in host memory
            host = batch.result.tolist()
        else:
            sess.tokens[:n].copy_(batch.staging, non_blocking=True)    # this step's inputs, host → device
            logits = sess.step(advance_on_device=False)            # the sampling kernel moves the positions on
            out = sampler.sample(logits[:n], list(range(n)), next_pos=sess.tok_pos, row_slot=sess.tok_slot)
            host = out.tolist()                                    # this step's result, device → host; synchronises
        self.h2d_bytes += 4 * n
        self.d2h_bytes += 4 * n
        self.decode_steps += 1
        return [host[r] for r in rows]

    def close_row(self, batch: _Batch, row: int) -> None:
        if batch.session is not None:
            batch.session.end_row(row)
        self.engine.end_sequence(batch.slots[row])
