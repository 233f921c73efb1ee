"""A levelled logger to stderr, and optional timers around kernel calls.

    VLRF_B200_LOG=error|warn|info|debug      what is printed (default warn)
    VLRF_B200_TIMERS=1                       time every kernel entry point with CUDA events, by kind

The reference prints its load and timing lines to stderr unconditionally (include/model/weights.hpp:266-269,
tools/vlrf_cli.cpp:301-313); here they are `info` lines.  With the timers on, every call into the kernel library
is bracketed by a pair of CUDA events on the current stream, and `timers.report()` gives, per entry point, the
number of calls and the device time between the events (each call is synchronised then, so the figures are for
reading, not for speed; captured graphs are launched plainly meanwhile).  NVTX ranges are pushed around the same
calls when torch has them, so a timeline shows the kernels under their entry points' names.
"""
from __future__ import annotations

import os
import sys

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}


def _level_from_env() -> int:
    return LEVELS.get(os.environ.get("VLRF_B200_LOG", "warn").lower(), 1)


_level = _level_from_env()


def set_level(name: str) -> None:
    global _level
    if name not in LEVELS:
        raise ValueError(f"unknown log level '{name}'; one of {', '.join(LEVELS)}")
    _level = LEVELS[name]


def enabled(name: str) -> bool:
    return LEVELS[name] <= _level


def _say(name: str, msg: str) -> None:
    if LEVELS[name] <= _level:
        print(f"[vlrf_b200 {name}] {msg}", file=sys.stderr, flush=True)


def error(msg: str) -> None:
    _say("error", msg)


def warn(msg: str) -> None:
    _say("warn", msg)


def info(msg: str) -> None:
    _say("info", msg)


def debug(msg: str) -> None:
    _say("debug", msg)


class KernelTimers:
    """Device time per kernel entry point, when switched on (`VLRF_B200_TIMERS=1` or `timers.enable()`)."""

    def __init__(self):
        self.on = os.environ.get("VLRF_B200_TIMERS", "0") not in ("", "0")
        self.calls: dict[str, int] = {}
        self.ms: dict[str, float] = {}

    def enable(self, on: bool = True) -> None:
        self.on = on

    def reset(self) -> None:
        self.calls.clear()
        self.ms.clear()

    def timed(self, name: str, fn, *args):
        """Run fn(*args) between two events on the current stream and add the time to `name`."""
        import torch
        nvtx = getattr(torch.cuda, "nvtx", None)
        if nvtx is not None:
            nvtx.range_push(name)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        try:
            out = fn(*args)
        finally:
            e1.record()
            if nvtx is not None:
                nvtx.range_pop()
        if not torch.cuda.is_current_stream_capturing():
            e1.synchronize()
            self.calls[name] = self.calls.get(name, 0) + 1
            self.ms[name] = self.ms.get(name, 0.0) + e0.elapsed_time(e1)
        return out

    def report(self) -> list:
        """[(entry point, calls, total ms, mean µs)] by total time, largest first."""
        rows = [(k, self.calls[k], self.ms[k], 1e3 * self.ms[k] / self.calls[k]) for k in self.calls]
        return sorted(rows, key=lambda r: -r[2])

    def table(self) -> str:
        rows = self.report()
        total = sum(r[2] for r in rows) or 1.0
        lines = [f"{'entry point':34} {'calls':>8} {'ms':>10} {'mean us':>9} {'share':>6}"]
        lines += [f"{k:34} {n:8d} {ms:10.3f} {us:9.2f} {100 * ms / total:5.1f}%" for k, n, ms, us in rows]
        return "\n".join(lines)


timers = KernelTimers()
