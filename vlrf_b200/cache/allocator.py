"""Host-side bookkeeping of the cache: which slots and which blocks are held.

`FreeList` hands out integer ids and takes them back, and refuses an id that is not held (freed
twice, or never given).  Nothing here touches the device, so the invariants (nothing lost, nothing
held twice, nothing freed twice) are tested without one.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    """The cache cannot do what was asked: it is full, or an id is misused."""


class FreeList:
    def __init__(self, n: int, what: str = "id"):
        if n < 0:
            raise CacheError(f"cannot make a list of {n} {what}s")
        self.n = n
        self.what = what
        # a stack, lowest ids on top: what was given back last is taken next, so reuse is immediate
        self._free = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self, k: int = 1) -> list[int]:
        if k < 0:
            raise CacheError(f"cannot take {k} {self.what}s")
        if k > len(self._free):
            raise CacheError(f"out of {self.what}s: {k} wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(k)]
        for i in out:
            self._held[i] = True
        return out

    def give(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if not (0 <= i < self.n):
                raise CacheError(f"{self.what} {i} does not exist (0…{self.n - 1})")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} is given back but is not held")
            self._held[i] = False  # marks duplicates inside `ids` too
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def held(self) -> list[int]:
        return [i for i, h in enumerate(self._held) if h]

    def check(self) -> None:
        """Every id is either free exactly once or held, never both."""
        seen = [0] * self.n
        for i in self._free:
            seen[i] += 1
        for i in range(self.n):
            if seen[i] > 1:
                raise CacheError(f"{self.what} {i} is on the free list {seen[i]} times")
            if seen[i] == 1 and self._held[i]:
                raise CacheError(f"{self.what} {i} is both free and held")
            if seen[i] == 0 and not self._held[i]:
                raise CacheError(f"{self.what} {i} is lost: neither free nor held")
