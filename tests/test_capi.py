"""The C interface (vlrf_b200/capi/vlrf_b200.h): from a C++ program on the device, and its host side here.

The C library forwards to the package's own entry point, so these tests are about the forwarding: arguments and
buffers across the boundary, status codes, and that a C++ program gets from a model folder to tokens that the plain
implementation also gives."""
import ctypes
import subprocess
import sysconfig

import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_F32


def built():
    from vlrf_b200.capi import build
    return build()


def lcg_ids(vocab, lens, seed):
    """The ids that tests/capi_program.cpp draws."""
    x, out = seed, []
    for n in lens:
        ids = []
        for _ in range(n):
            x = (x * 6364136223846793005 + 1442695040888963407) % 2 ** 64
            ids.append((x >> 33) % vocab)
        out.append(ids)
    return out


def test_the_library_joins_a_running_interpreter_and_maps_failures_to_statuses(tmp_path):
    from vlrf_b200.capi import bridge
    lib_path, cli = built()
    lib = ctypes.CDLL(str(lib_path))
    lib.vlrf_b200_create_model.restype = ctypes.c_void_p
    lib.vlrf_b200_last_error.restype = ctypes.c_char_p
    lib.vlrf_b200_status_str.restype = ctypes.c_char_p
    lib.vlrf_b200_load_dir.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int32, ctypes.c_int32]
    lib.vlrf_b200_get_info.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.vlrf_b200_free_model.argtypes = [ctypes.c_void_p]
    lib.vlrf_b200_presets.argtypes = [ctypes.c_char_p, ctypes.c_int32]
    lib.vlrf_b200_write_random_model.argtypes = [ctypes.c_char_p, ctypes.c_uint32, ctypes.c_char_p]
    lib.vlrf_b200_describe_dir.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int32]
    lib.vlrf_b200_default_sampling.argtypes = [ctypes.c_void_p]
    m = lib.vlrf_b200_create_model()
    assert m
    info = bridge.ModelInfo()
    assert lib.vlrf_b200_get_info(m, ctypes.byref(info)) == bridge.NOT_INIT
    assert lib.vlrf_b200_load_dir(m, str(tmp_path / "nothing").encode(), b"bfloat16", 0, 0) == bridge.IO
    assert b"nothing" in lib.vlrf_b200_last_error()
    assert lib.vlrf_b200_load_dir(None, b"x", b"bfloat16", 0, 0) == bridge.INVALID_ARG
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text('{"model_type": "no_such_architecture"}')
    assert lib.vlrf_b200_load_dir(m, str(bad).encode(), b"bfloat16", 0, 0) == bridge.BAD_MODEL
    assert b"registered" in lib.vlrf_b200_last_error()
    buf = ctypes.create_string_buffer(4096)
    assert lib.vlrf_b200_presets(buf, 4096) == 0 and b"tiny-a" in buf.value and b"gpt2-xl" in buf.value
    assert lib.vlrf_b200_presets(buf, 3) == bridge.INVALID_ARG                  # a buffer too small is refused, not overrun
    out = tmp_path / "made"
    assert lib.vlrf_b200_write_random_model(b"tiny-a", 5, str(out).encode()) == 0
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    assert lib.vlrf_b200_describe_dir(str(out).encode(), buf, 4096) == 0 and b"parameters: 141,056" in buf.value
    assert lib.vlrf_b200_write_random_model(b'{"model_type": "gpt2"}', 5, str(out).encode()) == bridge.BAD_MODEL
    s = bridge.Sampling()
    lib.vlrf_b200_default_sampling(ctypes.byref(s))
    assert (s.max_new_tokens, s.top_k, s.use_sampling, s.seed, s.n_stop_ids) == (128, 50, 1, 42, -1)
    assert abs(s.temperature - 0.8) < 1e-6 and abs(s.top_p - 0.9) < 1e-6 and s.repetition_penalty == 1.0
    assert lib.vlrf_b200_status_str(bridge.CTX_FULL) and lib.vlrf_b200_status_str(12345) == b"unknown error"
    lib.vlrf_b200_free_model(m)
    # the C++ command line, which hosts its own interpreter: the commands that need no device
    made = tmp_path / "cli_made"
    r = subprocess.run([str(cli), "init", "--config", "tiny-b", "--out", str(made), "--seed", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and (made / "model.safetensors").exists(), r.stderr
    r = subprocess.run([str(cli), "info", "--model", str(made)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and '"n_embd": 96' in r.stdout and "parameters: 419,232" in r.stdout
    r = subprocess.run([str(cli), "info", "--model", str(tmp_path / "nothing")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "file cannot be read" in r.stderr
    r = subprocess.run([str(cli), "run", "--model", str(made)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 2 and "--prompt" in r.stderr


def compile_program(tmp_path):
    from vlrf_b200.capi import SRC_DIR
    lib_path, _ = built()
    exe = tmp_path / "capi_program"
    libdir = sysconfig.get_config_var("LIBDIR")
    subprocess.run(["g++", "-O1", "-std=c++17", f"-I{SRC_DIR}", str(__import__("pathlib").Path(__file__).parent / "capi_program.cpp"),
                    "-o", str(exe), f"-L{lib_path.parent}", "-lvlrf_b200", f"-Wl,-rpath,{lib_path.parent}", f"-Wl,-rpath,{libdir}"],
                   check=True)
    return exe


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_cpp_program_loads_a_folder_and_generates_what_the_plain_implementation_does(tmp_path, model_dirs, plain_models, dtype):
    from vlrf_b200.capi import bridge
    cfg, w = plain_models["tiny_b"]
    exe = compile_program(tmp_path)
    lens, max_new, seed = [9, 1, 40, 100, 3], 24, 17
    r = subprocess.run([str(exe), str(model_dirs["tiny_b"]), dtype, "2", str(max_new), ",".join(map(str, lens)), str(seed)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln.split() for ln in r.stdout.splitlines()]
    got = {ln[0] + ("_" + ln[1] if ln[0] in ("gen", "status") else ""): ln[1:] for ln in lines}
    assert got["sizes"] == [str(ctypes.sizeof(bridge.Sampling)), str(ctypes.sizeof(bridge.ModelInfo))]
    assert got["info"] == [str(v) for v in (1000, 256, 96, 3, 512, 2, 1, 2)]
    prompts = lcg_ids(1000, lens, seed)
    tol = TOL_F32 if dtype == "float32" else 3e-2
    for i, p in enumerate(prompts):
        reason, ids = int(got[f"gen_{i}"][1]), [int(t) for t in got[f"gen_{i}"][2:]]
        assert reason == 1 and len(ids) == max_new
        if dtype == "float32":
            assert ids == plain.greedy_generate(cfg, w, p, max_new)
        else:
            seq = list(p)
            for t in ids:
                lg = plain.logits_all_positions(cfg, w, seq)[-1]
                assert float(lg.max() - lg[t]) <= 2 * tol * float(lg.abs().max())
                seq.append(t)
    truth = plain.logits_all_positions(cfg, w, prompts[0])[-1]
    if dtype == "float32":
        assert abs(float(got["logits"][0]) - float(truth.sum())) < 1e-2 and int(got["logits"][1]) == int(truth.argmax())
    assert float(got["step"][0]) <= (2e-4 if dtype == "float32" else 0.3)         # the same logits through single steps
    assert got["status_info_before_load"] == ["info_before_load", str(bridge.NOT_INIT)]
    assert got["status_load_missing"] == ["load_missing", str(bridge.IO)]
    assert got["status_step_bad_token"] == ["step_bad_token", str(bridge.INVALID_ARG)]
    assert got["status_step_freed_slot"] == ["step_freed_slot", str(bridge.INVALID_ARG)]
    assert got["status_too_long"] == ["too_long", str(bridge.CTX_FULL)]
    assert int(got["cache_bytes"][0]) > 0


@pytest.mark.gpu
def test_the_cpp_command_line_generates_what_the_python_one_does(tmp_path, model_dirs):
    import sys
    _, cli = built()
    f = tmp_path / "prompts.txt"
    f.write_text("5 17 3 900 44\n7\n1,2,3,4,5,6,7,8,9,10,11,12\n")
    args = ["run", "--model", str(model_dirs["tiny_b"]), "--prompts-file", str(f), "--tokens", "10", "--greedy", "--dtype", "float32"]
    a = subprocess.run([str(cli)] + args, capture_output=True, text=True, timeout=600)
    b = subprocess.run([sys.executable, "-m", "vlrf_b200.cli"] + args, capture_output=True, text=True, timeout=600,
                       cwd=str(__import__("pathlib").Path(__file__).parent.parent))
    assert a.returncode == 0 and b.returncode == 0, (a.stderr[-1000:], b.stderr[-1000:])

    def outputs(text):
        lines = text.splitlines()
        return [lines[i + 1] for i, ln in enumerate(lines) if ln.startswith("--- Output")]

    assert outputs(a.stdout) == outputs(b.stdout) and len(outputs(a.stdout)) == 3
