"""The cache of the sequences being served.

A sequence holds one *slot* from its first step to its end.  What a layer keeps per sequence is said
by its mixer as a *need*:

  KVNeed     keys and values per token: all of them (kind "full") or the last `window` (kind "window")
  StateNeed  a state of fixed size per sequence (for mixers that carry one)

Layers with equal needs form a *group* with storage of its own.  A key/value group owns a pool of
blocks of `block_tokens` tokens, K and V of shape [layer in group, block, kv_head, block_tokens,
head_dim], and a table [slot, block index] → block; blocks are taken as a sequence grows and go back
to the pool when it ends (for a window group, also once they lie wholly before the window).  A state
group owns [layer in group, slot, *shape], zeroed when a slot is taken.  `max_tokens` sizes every
key/value pool: it is the most tokens that live sequences hold at one time, each sequence's count
rounded up to whole blocks.

The reference keeps one sequence: a [max_seq, kv_heads·head_dim] store per layer with one `used`
counter (include/model/kv_cache.hpp:132-138, :215-251) that is re-laid out per head on every call
(include/model/attention.hpp:154-156); here the per-head layout is the stored one.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from .allocator import CacheError, FreeList

BLOCK_TOKENS = 64


@dataclasses.dataclass(frozen=True)
class KVNeed:
    n_kv_heads: int
    head_dim: int
    kind: str = "full"      # "full" | "window"
    window: int = 0         # for kind "window": a query sees the last `window` keys, itself included


@dataclasses.dataclass(frozen=True)
class StateNeed:
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass
class CacheView:
    """What one layer's mixer gets: its part of its group's storage."""
    need: object
    k: torch.Tensor | None = None            # [block, kv_head, block_tokens, head_dim]
    v: torch.Tensor | None = None
    block_table: torch.Tensor | None = None  # device int32 [slot, block index]
    state: torch.Tensor | None = None        # [slot, *shape]


class _KVGroup:
    def __init__(self, need: KVNeed, entries, n_blocks, n_slots, max_blocks, dtype, device):
        self.need, self.entries = need, list(entries)
        self.pool = FreeList(n_blocks, "cache block")
        shape = (len(self.entries), n_blocks, need.n_kv_heads, BLOCK_TOKENS, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        # the host's copy of the table lies in pinned memory where there is a GPU, so that bringing the device's
        # copy up to date is an asynchronous copy; `before_write` waits for a copy still reading it
        self._pinned = None
        if torch.device(device).type == "cuda":
            self._pinned = torch.full((n_slots, max_blocks), -1, dtype=torch.int32, pin_memory=True)
            self.table_host = self._pinned.numpy()
        else:
            self.table_host = np.full((n_slots, max_blocks), -1, dtype=np.int32)
        self.table_dev = torch.full((n_slots, max_blocks), -1, dtype=torch.int32, device=device)
        self.dirty = False
        self._copied = None            # event behind the latest copy of the table, while it may still be running

    def before_write(self) -> None:
        """Call before changing `table_host`: a copy to the device that is still under way reads it."""
        if self._copied is not None:
            self._copied.synchronize()
            self._copied = None
        self.dirty = True

    def sync(self) -> None:
        if not self.dirty:
            return
        if self._pinned is not None:
            self.table_dev.copy_(self._pinned, non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()
        else:
            self.table_dev.copy_(torch.from_numpy(self.table_host), non_blocking=False)
        self.dirty = False

    def blocks_of(self, slot) -> list[int]:
        row = self.table_host[slot]
        return [int(b) for b in row if b >= 0]

    def missing_for(self, slot, cur_len, new_len) -> list[int]:
        """Block indices that the queries at positions cur_len…new_len−1 need and the slot does not hold."""
        first = 0
        if self.need.kind == "window" and self.need.window > 0:
            first = max(0, cur_len + 1 - self.need.window) // BLOCK_TOKENS  # oldest key the first query sees
        last = (new_len + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        row = self.table_host[slot]
        return [i for i in range(first, last) if row[i] < 0]


class _StateGroup:
    def __init__(self, need: StateNeed, entries, n_slots, device):
        self.need, self.entries = need, list(entries)
        self.state = torch.zeros((len(self.entries), n_slots, *need.shape), dtype=need.dtype, device=device)


class SequenceCache:
    def __init__(self, needs, *, max_tokens: int, max_seq_len: int, dtype: torch.dtype, device,
                 n_slots: int | None = None):
        """needs: for every cache entry (one per layer execution that keeps something) its need, or None."""
        if max_tokens <= 0 or max_seq_len <= 0:
            raise CacheError("max_tokens and max_seq_len must be positive")
        self.block_tokens = BLOCK_TOKENS
        self.max_seq_len = max_seq_len
        self.n_blocks = (max_tokens + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        self.max_tokens = self.n_blocks * BLOCK_TOKENS
        # every live sequence holds at least one block, so there are never more sequences than blocks
        self.n_slots = n_slots if n_slots is not None else self.n_blocks
        self.max_blocks = (max_seq_len + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        self.device = torch.device(device)
        self.dtype = dtype
        self.slots = FreeList(self.n_slots, "cache slot")
        self.lengths = [0] * self.n_slots
        self.needs = list(needs)
        self._groups: list = []
        self._where: dict[int, tuple] = {}
        by_need: dict = {}
        for entry, need in enumerate(self.needs):
            if need is None:
                continue
            by_need.setdefault(need, []).append(entry)
        for need, entries in by_need.items():
            if isinstance(need, KVNeed):
                if need.kind not in ("full", "window"):
                    raise CacheError(f"unknown key/value need kind '{need.kind}'")
                if need.kind == "window" and need.window <= 0:
                    raise CacheError("a window need has a positive window")
                g = _KVGroup(need, entries, self.n_blocks, self.n_slots, self.max_blocks, dtype, self.device)
            elif isinstance(need, StateNeed):
                g = _StateGroup(need, entries, self.n_slots, self.device)
            else:
                raise CacheError(f"unknown cache need {need!r}")
            self._groups.append(g)
            for i, entry in enumerate(entries):
                self._where[entry] = (g, i)

    # -- storage ------------------------------------------------------------------------------
    def view(self, entry: int) -> CacheView:
        if entry not in self._where:
            raise CacheError(f"cache entry {entry} keeps nothing")
        g, i = self._where[entry]
        if isinstance(g, _KVGroup):
            return CacheView(g.need, k=g.k[i], v=g.v[i], block_table=g.table_dev)
        return CacheView(g.need, state=g.state[i])

    def bytes(self) -> int:
        total = 0
        for g in self._groups:
            if isinstance(g, _KVGroup):
                total += 2 * g.k.numel() * g.k.element_size()
            else:
                total += g.state.numel() * g.state.element_size()
        return total

    def live_kv_bytes(self, slots) -> int:
        """Bytes of keys and values that attention over `slots` reads at their present lengths."""
        total = 0
        for g in self._groups:
            if isinstance(g, _KVGroup):
                per_tok = 2 * len(g.entries) * g.need.n_kv_heads * g.need.head_dim * g.k.element_size()
                for s in slots:
                    n = self.lengths[s]
                    if g.need.kind == "window":
                        n = min(n, g.need.window)
                    total += n * per_tok
        return total

    # -- sequences ----------------------------------------------------------------------------
    def acquire(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for g in self._groups:
            if isinstance(g, _StateGroup):
                g.state[:, slot].zero_()   # a state is read before it is written
        return slot

    def _check_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"cache slot {slot} is not held by a sequence")

    def reserve(self, slot: int, new_len: int) -> None:
        """Make room for positions < new_len.  Either every group gets its blocks or nothing changes."""
        self._check_slot(slot)
        if new_len > self.max_seq_len:
            raise CacheError(f"a sequence of {new_len} tokens exceeds the {self.max_seq_len} positions of the model")
        kv = [g for g in self._groups if isinstance(g, _KVGroup)]
        wanted = [g.missing_for(slot, self.lengths[slot], new_len) for g in kv]
        for g, idx in zip(kv, wanted):
            if len(idx) > g.pool.n_free:
                held = g.pool.n_held * BLOCK_TOKENS
                raise CacheError(
                    f"cache full: {len(idx)} more block(s) of {BLOCK_TOKENS} tokens wanted, "
                    f"{g.pool.n_free} free ({held} of {self.max_tokens} tokens held)")
        for g, idx in zip(kv, wanted):
            if not idx:
                continue
            g.before_write()
            for i, b in zip(idx, g.pool.take(len(idx))):
                g.table_host[slot, i] = b

    def advance(self, slot: int, n_tokens: int) -> None:
        self._check_slot(slot)
        new_len = self.lengths[slot] + n_tokens
        if new_len > self.max_seq_len:
            raise CacheError(f"slot {slot}: {new_len} tokens exceed {self.max_seq_len} positions")
        self.lengths[slot] = new_len
        for g in self._groups:
            if isinstance(g, _KVGroup) and g.need.kind == "window":
                # blocks wholly before the window of the next query go back to the pool
                keep_from = max(0, new_len + 1 - g.need.window) // BLOCK_TOKENS
                row = g.table_host[slot]
                old = [int(row[i]) for i in range(keep_from) if row[i] >= 0]
                if old:
                    g.before_write()
                    row[:keep_from] = -1
                    g.pool.give(old)

    def release(self, slot: int) -> None:
        self._check_slot(slot)
        for g in self._groups:
            if isinstance(g, _KVGroup):
                blocks = g.blocks_of(slot)
                if blocks:
                    g.before_write()
                    g.pool.give(blocks)
                    g.table_host[slot, :] = -1
        self.lengths[slot] = 0
        self.slots.give([slot])

    def sync_tables(self) -> None:
        """Bring the device's block tables up to date (a copy on the current stream)."""
        for g in self._groups:
            if isinstance(g, _KVGroup):
                g.sync()

    # -- invariants ---------------------------------------------------------------------------
    def check(self) -> None:
        self.slots.check()
        for g in self._groups:
            if not isinstance(g, _KVGroup):
                continue
            g.pool.check()
            seen: dict[int, int] = {}
            for slot in range(self.n_slots):
                for b in g.blocks_of(slot):
                    if not self.slots.is_held(slot):
                        raise CacheError(f"free slot {slot} still maps block {b}")
                    if b in seen:
                        raise CacheError(f"block {b} is mapped by slots {seen[b]} and {slot}")
                    if not g.pool.is_held(b):
                        raise CacheError(f"slot {slot} maps block {b}, which the pool thinks free")
                    seen[b] = slot
            if len(seen) != g.pool.n_held:
                raise CacheError(f"{g.pool.n_held - len(seen)} block(s) are held but mapped by no slot")
