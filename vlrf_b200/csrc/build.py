"""Compiling the CUDA sources of this folder into one shared library for sm_100a.

`ensure_built()` compiles what is missing or stale (by a hash of the sources and flags) with nvcc,
object files in parallel, and returns the path of the library.  The build folder is `_build/` beside
the sources when that is writable, else `$VLRF_B200_BUILD_DIR`, else a per-user folder under the
system's temporary directory; nothing depends on HOME.  While compiling, a line is printed to stderr for
every file so that a first call in a fresh checkout shows progress.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

SRC_DIR = Path(__file__).parent
LIB_NAME = "libvlrf_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# VLRF_B200_KERNEL_TRACE=1: the decode step's kernels are compiled with time stamps at the stations of their critical
# path (see common.cuh); such a build is a measuring instrument, not the product, and is kept in a folder of its own
KERNEL_TRACE = os.environ.get("VLRF_B200_KERNEL_TRACE", "0") not in ("", "0")
if KERNEL_TRACE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DVLRF_KERNEL_TRACE"]


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(SRC_DIR.glob("*.cuh")) + list(SRC_DIR.glob("*.h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH): the CUDA kernels cannot be compiled, "
                       "and this framework has no other execution path")


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("VLRF_B200_BUILD_DIR")
    if env:
        d = Path(env)
        if _writable(d):
            return d
        raise RuntimeError(f"VLRF_B200_BUILD_DIR={env} is not writable")
    d = SRC_DIR / ("_build_trace" if KERNEL_TRACE else "_build")
    if _writable(d):
        return d
    d = Path(tempfile.gettempdir()) / f"vlrf_b200_build_{os.getuid()}"
    if _writable(d):
        return d
    raise RuntimeError("no writable folder to build the CUDA kernels in; set VLRF_B200_BUILD_DIR")


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[vlrf_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path) -> tuple[Path, float, str]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src, time.time() - t0, proc.stderr


def ensure_built(verbose: bool = True, force: bool = False) -> Path:
    out = build_dir()
    with open(out / ".lock", "w") as lock:  # one builder at a time; the others wait and find it built
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _ensure_built_locked(out, verbose, force)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _ensure_built_locked(out: Path, verbose: bool, force: bool) -> Path:
    lib = out / LIB_NAME
    srcs, hdrs = sources(), _headers()
    flags = " ".join(ARCH_FLAGS + NVCC_FLAGS)
    hdr_digest = _digest(hdrs, flags)
    stale = []
    for s in srcs:
        obj, stamp = out / (s.stem + ".o"), out / (s.stem + ".stamp")
        want = _digest([s], hdr_digest)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != want:
            stale.append((s, obj, stamp, want))
    lib_stamp = out / (LIB_NAME + ".stamp")
    lib_want = _digest(srcs, hdr_digest)
    if not stale and lib.exists() and lib_stamp.exists() and lib_stamp.read_text() == lib_want:
        return lib
    nvcc = find_nvcc()
    if verbose and stale:
        _say(f"compiling {len(stale)} CUDA source file(s) for sm_100a into {out} (first call only)")
    t0 = time.time()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(stale)))) as pool:
        futs = {pool.submit(_compile_one, nvcc, s, obj): (s, stamp, want) for s, obj, stamp, want in stale}
        pending = set(futs)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=10.0)
            for f in done:
                src, dt, _ = f.result()
                s, stamp, want = futs[f]
                stamp.write_text(want)
                if verbose:
                    _say(f"  {src.name} compiled in {dt:.1f} s")
            if pending and verbose:
                _say(f"  still compiling {len(pending)} file(s), {time.time() - t0:.0f} s so far")
    objs = [str(out / (s.stem + ".o")) for s in srcs]
    tmp = out / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *objs]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)  # atomic: another process never sees a half-written library
    lib_stamp.write_text(lib_want)
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.1f} s")
    return lib


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv))
