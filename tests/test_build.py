"""The kernel library's builder on a stand-in source folder (nvcc cross-compiles here without a GPU): a first
call compiles, a second finds everything up to date, a changed header makes every source stale, and without a
compiler the failure says so."""
import shutil

import pytest

from vlrf_b200.csrc import build

needs_nvcc = pytest.mark.skipif(shutil.which("nvcc") is None and not __import__("os").path.exists("/usr/local/cuda/bin/nvcc"),
                                reason="no nvcc on this machine")


@pytest.fixture
def tiny_sources(tmp_path, monkeypatch):
    src = tmp_path / "src"
    src.mkdir()
    (src / "answer.cuh").write_text("#pragma once\n#define ANSWER 41\n")
    (src / "one.cu").write_text('#include "answer.cuh"\nextern "C" int tiny_answer() { return ANSWER; }\n')
    (src / "two.cu").write_text('__global__ void tiny_kernel(int* p) { *p = 1; }\nextern "C" int tiny_two() { return 2; }\n')
    monkeypatch.setattr(build, "SRC_DIR", src)
    monkeypatch.setattr(build, "LIB_NAME", "libtiny.so")
    monkeypatch.setenv("VLRF_B200_BUILD_DIR", str(tmp_path / "out"))
    return src


@needs_nvcc
def test_first_call_compiles_then_nothing_until_a_source_or_header_changes(tiny_sources, capsys, monkeypatch):
    import ctypes
    lib = build.ensure_built()
    err = capsys.readouterr().err
    assert "compiling 2 CUDA source file(s) for sm_100a" in err and "built libtiny.so" in err
    assert ctypes.CDLL(str(lib)).tiny_answer() == 41
    # up to date: no compiler is even looked for
    monkeypatch.setattr(build, "find_nvcc", lambda: (_ for _ in ()).throw(AssertionError("nothing to compile")))
    assert build.ensure_built() == lib and capsys.readouterr().err == ""
    monkeypatch.undo()
    monkeypatch.setattr(build, "SRC_DIR", tiny_sources)
    monkeypatch.setattr(build, "LIB_NAME", "libtiny.so")
    monkeypatch.setenv("VLRF_B200_BUILD_DIR", str(lib.parent))
    # one source changes: only that one is compiled again
    (tiny_sources / "two.cu").write_text('extern "C" int tiny_two() { return 3; }\n')
    build.ensure_built()
    assert "compiling 1 CUDA source file(s)" in capsys.readouterr().err
    # a header changes: every source that may include it is stale
    (tiny_sources / "answer.cuh").write_text("#pragma once\n#define ANSWER 42\n")
    build.ensure_built()
    assert "compiling 2 CUDA source file(s)" in capsys.readouterr().err


def test_without_a_compiler_the_failure_says_what_is_missing(tiny_sources, monkeypatch):
    monkeypatch.setenv("NVCC", "/nowhere/nvcc")
    monkeypatch.setattr(build.shutil, "which", lambda name: None)
    # (the third place it looks, the toolkit's own folder, exists on this machine: hide every file called nvcc)
    monkeypatch.setattr(build.Path, "exists", lambda self: False if self.name == "nvcc" else type(self).is_file(self) or type(self).is_dir(self))
    with pytest.raises(RuntimeError, match="nvcc not found.*no other execution path"):
        build.ensure_built()


def test_a_build_folder_that_cannot_be_written_is_an_error_not_a_silent_fallback(tmp_path, monkeypatch):
    blocked = tmp_path / "file_in_the_way"
    blocked.write_text("")
    monkeypatch.setenv("VLRF_B200_BUILD_DIR", str(blocked / "sub"))
    with pytest.raises(RuntimeError, match="is not writable"):
        build.build_dir()


@needs_nvcc
def test_a_source_that_does_not_compile_reports_the_compilers_words(tiny_sources, capsys):
    (tiny_sources / "one.cu").write_text("this is not CUDA\n")
    with pytest.raises(RuntimeError, match="nvcc failed on one.cu"):
        build.ensure_built()
