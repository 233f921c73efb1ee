"""The C interface of the library (vlrf_b200.h), its implementation and the C++ command line over it.

`build()` compiles `libvlrf_b200.so` and `vlrf_b200_cli` with g++ against the running interpreter's headers and
library; both land in `_build/` beside the sources (or where `VLRF_B200_BUILD_DIR` says).  The C library forwards
to `bridge.py`, which hands over to the package's Python entry point: one engine, two ways in.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

SRC_DIR = Path(__file__).parent
LIB_NAME = "libvlrf_b200.so"
CLI_NAME = "vlrf_b200_cli"


def build_dir() -> Path:
    env = os.environ.get("VLRF_B200_BUILD_DIR")
    d = Path(env) / "capi" if env else SRC_DIR / "_build"
    d.mkdir(parents=True, exist_ok=True)
    return d


def build(verbose: bool = False) -> tuple[Path, Path]:
    """(library, command line); compiled when missing or older than the sources."""
    cxx = os.environ.get("CXX") or shutil.which("g++")
    if cxx is None:
        raise RuntimeError("g++ not found: the C interface cannot be built")
    out = build_dir()
    lib, cli = out / LIB_NAME, out / CLI_NAME
    sources = [SRC_DIR / "vlrf_b200.h", SRC_DIR / "vlrf_b200_api.cpp", SRC_DIR / "vlrf_b200_cli.cpp"]
    home = str(SRC_DIR.parent.parent)
    digest = hashlib.sha256("".join(p.read_text() for p in sources).encode() + home.encode() + sys.executable.encode()).hexdigest()
    stamp = out / "capi.stamp"
    if lib.exists() and cli.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib, cli
    include = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR")
    pylib = "python" + sysconfig.get_config_var("LDVERSION")
    say = (lambda m: print(f"[vlrf_b200 build] {m}", file=sys.stderr, flush=True)) if verbose else (lambda m: None)
    say(f"compiling {LIB_NAME}")
    subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", f"-I{include}", f"-I{SRC_DIR}",
                    f'-DVLRF_B200_DEFAULT_HOME="{home}"', f'-DVLRF_B200_DEFAULT_PYTHON="{sys.executable}"',
                    str(SRC_DIR / "vlrf_b200_api.cpp"), "-o", str(lib), f"-L{libdir}", f"-l{pylib}", f"-Wl,-rpath,{libdir}",
                    "-lpthread", "-ldl"], check=True)
    say(f"compiling {CLI_NAME}")
    subprocess.run([cxx, "-O2", "-std=c++17", f"-I{SRC_DIR}", str(SRC_DIR / "vlrf_b200_cli.cpp"), "-o", str(cli), f"-L{out}",
                    "-lvlrf_b200", f"-Wl,-rpath,{out}", f"-Wl,-rpath,{libdir}"], check=True)
    stamp.write_text(digest)
    return lib, cli
