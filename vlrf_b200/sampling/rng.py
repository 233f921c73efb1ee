"""The counter-based random stream of a request, the same arithmetic as the sampling kernel.

A request's key depends on the call's seed and the request's index only; its n-th draw depends on the
key and n only.  So what a request samples does not depend on the batch it is in or the slot it holds.
(The reference keeps one mt19937 per model, seed 42: include/model/transformer.hpp:203.)
"""
from __future__ import annotations

_M = (1 << 64) - 1


def _mix64(x: int) -> int:
    x &= _M
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M
    x ^= x >> 31
    return x


def request_key(seed: int, request_index: int) -> int:
    """64-bit key of a request's stream."""
    return _mix64(_mix64(seed & _M) + 0x9E3779B97F4A7C15 * (request_index + 1))


def uniform01(key: int, counter: int) -> float:
    """The draw number `counter` of the stream `key`: 24 bits in [0, 1)."""
    x = _mix64(key + 0x9E3779B97F4A7C15 * ((counter + 1) & 0xFFFFFFFF))
    return (x >> 40) / 16777216.0


def as_signed64(key: int) -> int:
    """The key as torch.int64 holds it."""
    return key - (1 << 64) if key >= (1 << 63) else key
