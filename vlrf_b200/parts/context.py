"""What a step hands to the parts: the tokens of this step, where they sit, and scratch tensors.

A step runs a flat list of tokens.  Token t belongs to the sequence in cache slot `tok_slot[t]` and
sits at position `tok_pos[t]` of it; a slot of −1 marks a padding row that every part skips.  Parts
read nothing else about the batch, so the same code serves prompts of unequal lengths and single
decoded tokens.
"""
from __future__ import annotations

import dataclasses

import torch


class Workspace:
    """Named scratch tensors that live across steps, so steps allocate nothing once warm and a
    captured step sees stable addresses.  `get` returns a [rows, cols] view of the named buffer, which
    grows when a step asks for more than it holds."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._bufs: dict[str, torch.Tensor] = {}
        self._views: dict = {}   # (name, rows, cols, dtype) -> the view handed out last time (making one costs 2 to 3 us)
        self.frozen = False  # set while a captured graph depends on the addresses
        self.generation = 0  # counts (re)allocations: captured steps are valid for one generation only
        from ..csrc.ops import RowStats
        #: statistics of the residual rows that the step's last product wrote (see csrc.ops.RowStats); parts hand
        #: this to the products that may leave or use them, the block forgets them after parts it cannot vouch for
        self.row_stats = RowStats(self.device)

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, rows, cols, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        n = rows * cols
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace '{name}' would have to grow while a captured step uses it")
            cap = max(n, 1)
            if buf is not None and buf.dtype == dtype:
                cap = max(cap, 2 * buf.numel())
            buf = torch.empty(cap, dtype=dtype, device=self.device)
            self._bufs[name] = buf
            self.generation += 1
            self._views.clear()                  # views of the buffer that went
        if len(self._views) > 1024:
            self._views.clear()
        view = buf[:n].view(rows, cols)
        self._views[key] = view
        return view

    def get_zeroed(self, name: str, n: int, dtype: torch.dtype) -> torch.Tensor:
        """A flat buffer that is zero when first handed out (and again after it had to grow); whoever uses
        it leaves it zero."""
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace '{name}' would have to grow while a captured step uses it")
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = buf
            self.generation += 1
        return buf[:n]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclasses.dataclass
class StepContext:
    n_tokens: int                    # rows of this step, padding included
    tokens: torch.Tensor             # int32 [n_tokens]
    tok_slot: torch.Tensor           # int32 [n_tokens]; −1 = padding
    tok_pos: torch.Tensor            # int32 [n_tokens]
    n_seqs: int
    seq_slot: torch.Tensor           # int32 [n_seqs]
    seq_start: torch.Tensor          # int32 [n_seqs + 1]: first row of each sequence's tokens
    seq_pos0: torch.Tensor           # int32 [n_seqs]: tokens the sequence held before this step
    max_new: int                     # longest run of new tokens of one sequence (1 = a decode step)
    max_context: int                 # longest context after this step
    logit_rows: torch.Tensor         # int32 [n_logit_rows]: rows whose logits are wanted
    n_logit_rows: int
    act_dtype: torch.dtype           # dtype of activations between kernels
    dev_err: torch.Tensor            # int32 [1]: bits that kernels set instead of faulting
    ws: Workspace
    #: host copies for parts that plan on the host (e.g. tiling a prefill)
    host_seq_slots: list = dataclasses.field(default_factory=list)
    host_seq_lens: list = dataclasses.field(default_factory=list)
    host_seq_pos0: list = dataclasses.field(default_factory=list)
