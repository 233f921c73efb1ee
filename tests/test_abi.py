"""The ctypes table of `vlrf_b200.csrc` against the `extern "C"` definitions in the CUDA sources.

A wrong argument list in the table is not caught by the loader (ctypes cannot see C prototypes): a kernel
would get shifted arguments.  This test parses the definitions and compares count and kind of every argument.
"""
import ctypes
import re
from pathlib import Path

SRC = Path(__file__).resolve().parent.parent / "vlrf_b200" / "csrc"


def c_definitions() -> dict:
    """name -> (return type, [argument types]) of every `extern "C"` function defined in the sources."""
    out = {}
    for path in sorted(SRC.glob("*.cu")):
        text = re.sub(r"/\*.*?\*/", "", re.sub(r"//[^\n]*", "", path.read_text()), flags=re.S)
        for m in re.finditer(r'extern\s+"C"\s+([\w\s\*]+?)\s*\b(\w+)\s*\(([^)]*)\)\s*\{', text):
            ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
            kinds = []
            if args and args != "void":
                for a in args.split(","):
                    a = " ".join(a.split())
                    if "*" in a or a.startswith("cudaStream_t"):
                        kinds.append("pointer")
                    elif re.match(r"(const )?(unsigned )?(int|uint32_t)\b", a):
                        kinds.append("int")
                    elif re.match(r"(const )?float\b", a):
                        kinds.append("float")
                    elif re.match(r"(const )?(long long|unsigned long long|int64_t|uint64_t|size_t)\b", a):
                        kinds.append("int64")
                    else:
                        raise AssertionError(f"{path.name}: {name}: argument '{a}' of a kind this test does not know")
            assert name not in out, f"{name} is defined twice"
            out[name] = (ret, kinds)
    return out


KIND_OF = {ctypes.c_void_p: "pointer", ctypes.c_char_p: "pointer", ctypes.c_int: "int", ctypes.c_uint: "int",
           ctypes.c_float: "float", ctypes.c_longlong: "int64", ctypes.c_ulonglong: "int64", ctypes.c_size_t: "int64"}


def kind(t) -> str:
    if t in KIND_OF:
        return KIND_OF[t]
    if isinstance(t, type) and issubclass(t, ctypes._Pointer):
        return "pointer"
    raise AssertionError(f"ctypes type {t} of a kind this test does not know")


def test_every_entry_in_the_table_matches_its_definition():
    from vlrf_b200.csrc import _SIGNATURES
    defs = c_definitions()
    assert len(defs) >= 20
    for name, argtypes in _SIGNATURES.items():
        assert name in defs, f"{name} is in the ctypes table but no source defines it"
        ret, kinds = defs[name]
        assert [kind(t) for t in argtypes] == kinds, f"{name}: table {[kind(t) for t in argtypes]} against source {kinds}"
        # the loader gives every function of the table an int result
        assert ret == "int", f"{name} returns {ret}"


def test_every_entry_point_that_python_calls_exists():
    """Names given to `call("…")` or looked up on the loaded library (`library().…`, `lib.…`), here and in the
    tests: each must be defined in the sources."""
    defs = c_definitions()
    pattern = re.compile(r'(?:call\(\s*"|library\(\)\.|\blib\.)(vlrf_[a-z0-9_]+)')
    used = set()
    for path in list(SRC.parent.rglob("*.py")) + list(Path(__file__).resolve().parent.glob("*.py")):
        if path.name != Path(__file__).name:
            used |= set(pattern.findall(path.read_text()))
    assert len(used) >= 20
    # (names of the model-level C interface are held against its header; its definitions are C++, not in the table)
    capi = (SRC.parent / "capi" / "vlrf_b200_api.cpp").read_text()
    missing = sorted(u for u in used if u not in defs and not (u.startswith("vlrf_b200_") and re.search(rf"\b{u}\(", capi)))
    assert not missing, f"called from Python but defined in no source: {missing}"


def header_declarations() -> dict:
    """name -> (return type, [argument kinds]) of every prototype in the library's C header."""
    text = (SRC / "vlrf_b200_kernels.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", re.sub(r"//[^\n]*", "", text), flags=re.S)
    out = {}
    for m in re.finditer(r"^([\w\s\*]+?)\s*\b(vlrf_\w+)\s*\(([^)]*)\)\s*;", text, flags=re.M):
        ret, name, args = " ".join(m.group(1).split()), m.group(2), m.group(3).strip()
        kinds = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a or a.startswith("cudaStream_t"):
                    kinds.append("pointer")
                elif re.match(r"(const )?(unsigned )?int\b", a):
                    kinds.append("int")
                elif re.match(r"(const )?float\b", a):
                    kinds.append("float")
                else:
                    kinds.append("int64")
        out[name] = (ret, kinds)
    return out


def test_the_c_header_declares_exactly_what_the_sources_define():
    """`vlrf_b200_kernels.h` is what a C or C++ caller includes: every exported function, with the arguments of
    its definition, and nothing that does not exist."""
    defs, decl = c_definitions(), header_declarations()
    assert sorted(decl) == sorted(defs)
    for name, (ret, kinds) in defs.items():
        assert decl[name] == (ret, kinds), f"{name}: header {decl[name]} against source {(ret, kinds)}"
    # every source sees the header (through common.cuh), so the compiler holds each definition against it too
    assert '#include "vlrf_b200_kernels.h"' in (SRC / "common.cuh").read_text()
    for path in SRC.glob("*.cu"):
        assert '#include "common.cuh"' in path.read_text(), f"{path.name} does not include common.cuh"
