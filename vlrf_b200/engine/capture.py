"""Capturing a step's launches in a CUDA graph."""
from __future__ import annotations

import contextlib
import gc

import torch


@contextlib.contextmanager
def capture_into(graph: "torch.cuda.CUDAGraph"):
    """`torch.cuda.graph(graph)` with Python's garbage collector held off meanwhile.  A collection that
    happens to run in the middle of a capture may destroy CUDA objects of earlier batches that were waiting
    as cyclic garbage (graphs, events, pinned buffers); CUDA refuses that while a stream is capturing, and the
    error, raised inside a destructor, ends the process.  (torch collects once itself before it begins.)"""
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
    finally:
        if was_enabled:
            gc.enable()
