"""The CUDA kernels of the framework, loaded as one shared library through ctypes.

There is no other execution path: if the library cannot be compiled or loaded, or no CUDA device is
present, every operation raises `KernelError`.  The functions of `vlrf_b200.csrc.ops` take torch
tensors on the device, check them, and call the `extern "C"` entry points with raw pointers and the
current CUDA stream.
"""
from __future__ import annotations

import ctypes
import threading

from ..log import timers as _timers
from .build import ensure_built


class KernelError(RuntimeError):
    """A kernel refused its arguments, or the kernel library is unavailable."""


_lib = None
_lock = threading.Lock()

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

#: name -> argument types; every function returns int (0 = ok) unless noted
_SIGNATURES = {
    "vlrf_device_info": [ctypes.POINTER(_c_int)] * 4,
    "vlrf_embed": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                   _c_void_p, _c_void_p, _c_void_p],
    "vlrf_layernorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float,
                       _c_void_p],
    "vlrf_gemm_simt": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "vlrf_kv_append": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "vlrf_attn_generic": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                          _c_void_p, _c_void_p],
    "vlrf_set_chained_launch": [_c_int],
    "vlrf_trace_dims": [ctypes.POINTER(_c_int)] * 3,
    "vlrf_trace_read": [_c_void_p],
    "vlrf_gemm_skinny_ln_fits": [_c_int, _c_int],
    "vlrf_gemm_skinny": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                         _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_void_p, _c_void_p],
    "vlrf_gemm_splitk_takes": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "vlrf_gemm_splitk": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                         _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "vlrf_gemm_tcgen05_takes": [_c_int, _c_int, _c_int, _c_int],
    "vlrf_gemm_tcgen05": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "vlrf_attn_prefill_takes": [_c_int, _c_int, _c_int, _c_int],
    "vlrf_attn_prefill": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                          _c_int, _c_void_p, _c_void_p],
    "vlrf_attn_prefill_tc_takes": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "vlrf_gemm_tcgen05_force_width": [_c_int],
    "vlrf_attn_prefill_tc_part_floats": [],
    "vlrf_attn_prefill_tc_max_parts": [],
    "vlrf_attn_prefill_tc_min_part_blocks": [],
    "vlrf_attn_prefill_tc_tile": [],
    "vlrf_attn_prefill_tc": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                             _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "vlrf_attn_decode_needs_scratch": [_c_int, _c_int],
    "vlrf_attn_decode": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                         _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                         _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "vlrf_decode_program_op_bytes": [],
    "vlrf_decode_program_max_rows": [],
    "vlrf_decode_program_gemv_takes": [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int],
    "vlrf_decode_program_attention_takes": [_c_int, _c_int],
    "vlrf_decode_op_embed": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                             _c_int],
    "vlrf_decode_op_gemv": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                            _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                            _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_int],
    "vlrf_decode_op_attention": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                 _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                 _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_void_p],
    "vlrf_decode_program_run": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "vlrf_sample": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "vlrf_apply_penalties": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; built on first use.  Raises KernelError if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = ensure_built()
            lib = ctypes.CDLL(str(path))
        except Exception as exc:  # noqa: BLE001 - reported as the one error of this layer
            raise KernelError(f"the CUDA kernel library is unavailable: {exc}") from exc
        lib.vlrf_last_error.restype = ctypes.c_char_p
        lib.vlrf_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as exc:
                raise KernelError(f"the kernel library lacks the symbol {name}") from exc
            fn.argtypes = argtypes
            fn.restype = _c_int
        _lib = lib
        return lib


def register_signatures(extra: dict) -> None:
    """Add entry points (used by source files that join the library later)."""
    _SIGNATURES.update(extra)


_launches = 0


def launch_count() -> int:
    """How many kernel entry points have been called so far (each launches one kernel unless it says
    otherwise); replays of a captured graph are counted by whoever replays it."""
    return _launches


def call_host(name: str, *args) -> None:
    """An entry point that only works on the host (it launches nothing, so it is not counted as a launch)."""
    lib = library()
    status = getattr(lib, name)(*args)
    if status != 0:
        raise KernelError(f"{name}: {lib.vlrf_last_error().decode('utf-8', 'replace')} (status {status})")


def call(name: str, *args) -> None:
    global _launches
    lib = library()
    _launches += 1
    if _timers.on:
        status = _timers.timed(name, getattr(lib, name), *args)
    else:
        status = getattr(lib, name)(*args)
    if status != 0:
        raise KernelError(f"{name}: {lib.vlrf_last_error().decode('utf-8', 'replace')} (status {status})")
