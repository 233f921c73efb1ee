"""The generation loop's backend on the device: `Engine.step` plus the sampling kernels."""
from __future__ import annotations

import dataclasses

from ..sampling.rng import request_key
from ..sampling.sampler import RowSampler
from .step import Engine, StepEntry


@dataclasses.dataclass
class _Batch:
    slots: list
    sampler: RowSampler


class DeviceBackend:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def limits(self):
        c = self.engine.cache
        return c.max_tokens, c.n_slots, c.block_tokens, self.engine.model.max_seq_len

    def open_batch(self, requests: list) -> _Batch:
        slots = [self.engine.start_sequence() for _ in requests]
        keys = [request_key(r.params.seed, r.index) for r in requests]
        history = max((r.params.max_new_tokens for r in requests), default=1)
        sampler = RowSampler([r.params for r in requests], keys, self.engine.device, history)
        return _Batch(slots, sampler)

    def run(self, batch: _Batch, rows: list, tokens: list) -> list:
        entries = [StepEntry(batch.slots[r], toks, [len(toks) - 1]) for r, toks in zip(rows, tokens)]
        logits = self.engine.step(entries)
        out = batch.sampler.sample(logits, rows)
        host = out.tolist()                      # the step's one device→host read; synchronises
        self.h2d_bytes += 4 * (3 * sum(len(t) for t in tokens) + 4 * len(rows) + 1)
        self.d2h_bytes += 4 * len(rows)
        self.engine.check_device_errors()
        return host

    def close_row(self, batch: _Batch, row: int) -> None:
        self.engine.end_sequence(batch.slots[row])
