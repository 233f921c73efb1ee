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


#: what the stations of a kernel's time stamps mean, by kind of kernel (vlrf_b200/csrc: gemm_splitk.cu, attention_decode.cu)
TRACE_KINDS = {1: ("product", ["begins", "waited", "x in smem", "products", "sent", "received", "stored"]),
               2: ("attention", ["begins", "waited", "first chunk", "warp 0 done", "all warps", "", "stored"]),
               3: ("gemm", ["begins", "waited", "first tile", "last tile", "", "", "stored"]),
               4: ("attn", ["begins", "waited", "", "", "", "", "done"])}


def kernel_timeline() -> list:
    """The time stamps that the decode step's kernels left (a build with VLRF_B200_KERNEL_TRACE=1), one record per
    launch in launch order: {"launch", "kind", "ctas", "first": [...], "last": [...]}: per station the earliest and
    the latest CTA, in microseconds after the previous record's last stamp (the first record: after its own first).
    Reading clears the buffer.  A replayed graph leaves the stamps of its last replays."""
    import ctypes

    import numpy as np

    from .csrc import KernelError, call_host, library
    lib = library()
    dims = [ctypes.c_int(0) for _ in range(3)]
    lib.vlrf_trace_dims(*[ctypes.byref(d) for d in dims])
    slots, ctas, stations = (d.value for d in dims)
    if slots == 0:
        raise KernelError("this build of the kernels has no time stamps: set VLRF_B200_KERNEL_TRACE=1 before the first import")
    buf = np.zeros((slots, ctas, 2 + stations), dtype=np.int64)
    call_host("vlrf_trace_read", buf.ctypes.data_as(ctypes.c_void_p))
    records = []
    for s in range(slots):
        live = buf[s, :, 0] > 0
        if not live.any():
            continue
        launch = int(buf[s, live, 0].max())
        rows = buf[s][live & (buf[s, :, 0] == launch)]
        records.append((launch, int(rows[0, 1]), rows[:, 2:].astype(np.float64)))
    records.sort(key=lambda r: r[0])
    out, prev_end = [], None
    for launch, kind, t in records:
        seen = np.where(t > 0, t, np.nan)
        base = prev_end if prev_end is not None else np.nanmin(seen)
        first = [None if np.isnan(v) else round((v - base) / 1e3, 2) for v in np.nanmin(seen, axis=0)] if seen.size else []
        last = [None if np.isnan(v) else round((v - base) / 1e3, 2) for v in np.nanmax(seen, axis=0)] if seen.size else []
        out.append({"launch": launch, "kind": kind, "ctas": int(t.shape[0]), "first": first, "last": last})
        prev_end = np.nanmax(seen)
    return out


def timeline_table(records: list, last: int | None = None) -> str:
    """The records of `kernel_timeline` (the last `last` of them) as text: per launch and station, earliest…latest CTA
    in microseconds after the launch before it ended."""
    lines = []
    for r in (records[-last:] if last else records):
        name, stations = TRACE_KINDS.get(r["kind"], (f"kind {r['kind']}", [""] * 8))
        cells = []
        for i, label in enumerate(stations):
            if label and i < len(r["first"]) and r["first"][i] is not None:
                cells.append(f"{label} {r['first'][i]:6.2f}…{r['last'][i]:6.2f}")
        lines.append(f"{name:9} {r['ctas']:3d} CTAs | " + " | ".join(cells))
    return "\n".join(lines)
