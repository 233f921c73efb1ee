"""Choosing the next token of every row of logits on the device."""
from __future__ import annotations

import torch

from ..csrc import ops
from .rng import as_signed64


class RowSampler:
    """Per-row sampling state for a batch of requests, resident on the device.

    Row i holds request i's options, its random key and draw counter, and the tokens it has generated
    (for the penalties).  `sample(logits, rows)` picks one token for each listed row from the matching
    row of `logits`, appends it to the row's history, and returns the tokens as a device tensor.
    """

    def __init__(self, params: list, keys: list, device, max_history: int, *, any_sampling: bool | None = None,
                 any_penalties: bool | None = None):
        """`any_sampling` / `any_penalties`: what the rows must be able to do even if none of `params` asks for it
        now (rows are given to other requests later, see `set_row`); by default what `params` ask for."""
        n = len(params)
        self.n, self.device = n, torch.device(device)
        self.params = list(params)
        self.any_sampling = any(not p.greedy for p in params) if any_sampling is None else bool(any_sampling)
        self.any_penalties = any(p.has_penalties for p in params) if any_penalties is None else bool(any_penalties)
        f32 = lambda vals: torch.tensor(vals, dtype=torch.float32, device=self.device)  # noqa: E731
        i32 = lambda vals: torch.tensor(vals, dtype=torch.int32, device=self.device)    # noqa: E731
        self.temperature = f32([0.0 if p.greedy else p.temperature for p in params])
        self.top_k = i32([p.top_k for p in params])
        self.top_p = f32([p.top_p for p in params])
        self.rng_key = torch.tensor([as_signed64(k) for k in keys], dtype=torch.int64, device=self.device)
        self.rng_ctr = torch.zeros(n, dtype=torch.int32, device=self.device)
        if self.any_penalties:
            self.rep = f32([p.repetition_penalty for p in params])
            self.freq = f32([p.frequency_penalty for p in params])
            self.pres = f32([p.presence_penalty for p in params])
            self.ngram = i32([p.no_repeat_ngram_size for p in params])
            self.history = torch.zeros((n, max(1, max_history)), dtype=torch.int32, device=self.device)
            self.history_len = torch.zeros(n, dtype=torch.int32, device=self.device)
        self.out = torch.zeros(n, dtype=torch.int32, device=self.device)

    def set_row(self, row: int, params, key: int) -> None:
        """The row goes to another request: its options, a fresh random stream and an empty history.  The tensors stay
        where they are (a captured step reads them), only the row's entries change."""
        if (not params.greedy and not self.any_sampling) or (params.has_penalties and not self.any_penalties):
            raise ValueError("the sampler was set up without what this request's options need")
        self.params[row] = params
        self.temperature[row] = 0.0 if params.greedy else params.temperature
        self.top_k[row] = params.top_k
        self.top_p[row] = params.top_p
        self.rng_key[row] = as_signed64(key)
        self.rng_ctr[row] = 0
        if self.any_penalties:
            self.rep[row] = params.repetition_penalty
            self.freq[row] = params.frequency_penalty
            self.pres[row] = params.presence_penalty
            self.ngram[row] = params.no_repeat_ngram_size
            self.history_len[row] = 0

    def sample(self, logits: torch.Tensor, rows: list, *, next_pos=None, row_slot=None) -> torch.Tensor:
        """logits [len(rows), vocab] float32; rows: which requests these logits belong to, in order.
        `next_pos`, `row_slot`: a decode session's tables, advanced by the sampling kernel itself."""
        m = len(rows)
        all_rows = m == self.n and rows == list(range(self.n))
        idx = None if all_rows else torch.tensor(rows, dtype=torch.long, device=self.device)
        pick = (lambda t: t) if all_rows else (lambda t: t.index_select(0, idx))
        if self.any_penalties:
            ops.apply_penalties(logits, m, pick(self.history).contiguous(), pick(self.history_len).contiguous(),
                                repetition=pick(self.rep), frequency=pick(self.freq), presence=pick(self.pres),
                                no_repeat_ngram=pick(self.ngram))
        out = self.out[:m]
        if self.any_sampling:
            ctr = pick(self.rng_ctr).contiguous()
            ops.sample(logits, m, out, temperature=pick(self.temperature), top_k=pick(self.top_k),
                       top_p=pick(self.top_p), rng_key=pick(self.rng_key), rng_ctr=ctr, next_pos=next_pos,
                       row_slot=row_slot)
            if all_rows:
                pass  # the kernel advanced the counters in place
            else:
                self.rng_ctr.index_copy_(0, idx, ctr)
        else:
            ops.sample(logits, m, out, next_pos=next_pos, row_slot=row_slot)
        if self.any_penalties:
            r = torch.arange(self.n, device=self.device) if all_rows else idx
            # a row whose history is full overwrites its last entry and counts no further (rows that hold no request are
            # sampled along in a decode session and would count without end)
            at = self.history_len.index_select(0, r).long().clamp_(max=self.history.shape[1] - 1)
            self.history[r, at] = out.to(torch.int32)
            self.history_len.index_add_(0, r, torch.ones(m, dtype=torch.int32, device=self.device))
            self.history_len.clamp_(max=self.history.shape[1])
        return out
