#!/usr/bin/env python3
"""The reference arm of the benchmark: VLRF-org/VLRF's own CPU library, unmodified, timed through its C API.

    python baseline/reference_arm.py --steps K --warmup W [--batch 8]

What runs is the reference's stock path: its sources, copied as they are to `baseline/_ref/`, built into
`libvlrf.so` by its own CMakeLists.txt (the AVX2/FMA kernels switched on, as its README asks for), a GPT-2
checkpoint in its own `.nfw` format written by its own `tools/converter/nfw_writer.py`, its config.json
dialect (tools/converter/convert_gpt2.py:148-173), then `vlrf_create_model → vlrf_load_weights →
vlrf_generate_ids` (include/api/vlrf.h:116-200) and `vlrf_get_logits` for the prompt figure.  Only this
harness (random weights, token ids, clocks) is not the reference's.  Nothing of the vlrf_b200 package is
imported.

The reference holds one sequence and has no batch (include/model/transformer.hpp:439), so a batch of B is B
sequences one after another; the decoding rate is that of a single sequence.  It computes in float32 on the
host cores.  Both facts are named in the printed line (`same_config: false`).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BUILD = os.path.join(HERE, "_build")
LIB = os.path.join(BUILD, "libvlrf.so")
PROMPT_LEN = 512

# GPT-2 small layer sizes (the benchmark configuration); the reference's names for them
SIZES = dict(vocab_size=50257, d_model=768, d_ff=3072, n_heads=12, n_kv_heads=12, n_layers=12, max_seq_len=1024)


class Unavailable(Exception):
    pass


def ensure_sources() -> None:
    if os.path.isfile(os.path.join(REF, "CMakeLists.txt")):
        return
    src = os.environ.get("VLRF_REFERENCE_SRC", "/root/reference")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        raise Unavailable("no copy of the reference under baseline/_ref and none at " + src)
    shutil.copytree(src, REF, dirs_exist_ok=True)


def ensure_library() -> str:
    if os.path.isfile(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(os.path.join(REF, "CMakeLists.txt")):
        return LIB
    for tool in ("cmake", "g++"):
        if shutil.which(tool) is None:
            raise Unavailable(f"{tool} is not installed here, so the reference's library cannot be built")
    try:
        subprocess.run(["cmake", "-S", REF, "-B", BUILD, "-DCMAKE_BUILD_TYPE=Release", "-DVLRF_USE_AVX2=ON",
                        "-DVLRF_BUILD_TOOLS=OFF"], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
        subprocess.run(["cmake", "--build", BUILD, "--target", "vlrf", "-j", str(os.cpu_count() or 4)], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
    except subprocess.CalledProcessError as e:
        tail = (e.stderr or b"").decode(errors="replace").strip().splitlines()[-1:] or ["no message"]
        raise Unavailable("the reference's CMake build failed: " + tail[0][:160]) from None
    if not os.path.isfile(LIB):
        raise Unavailable("the reference's CMake build left no libvlrf.so")
    return LIB


def write_checkpoint(folder: str, n_layers: int, seed: int = 1234) -> str:
    """Random GPT-2 weights under the reference's tensor names (tools/converter/convert_gpt2.py:98-139),
    N(0, 0.02) matrices like its own random_init (include/model/transformer.hpp:566-629), written by its
    own writer; config.json in its dialect."""
    import numpy as np
    sys.path.insert(0, os.path.join(REF, "tools", "converter"))
    import nfw_writer
    rs = np.random.RandomState(seed)
    d, f, V, P = SIZES["d_model"], SIZES["d_ff"], SIZES["vocab_size"], SIZES["max_seq_len"]

    def n(*shape, std=0.02, mean=0.0):
        return (mean + std * rs.standard_normal(shape)).astype(np.float32)

    t = {"embed.weight": n(V, d), "pos_embed.weight": n(P, d), "ln_final.weight": n(d, mean=1.0), "ln_final.bias": n(d)}
    for i in range(n_layers):
        p = f"layers.{i}."
        for nm in "qkv":
            t[p + f"attn.{nm}_proj.weight"], t[p + f"attn.{nm}_proj.bias"] = n(d, d), n(d, std=0.01)
        t[p + "attn.o_proj.weight"], t[p + "attn.o_proj.bias"] = n(d, d), n(d, std=0.01)
        t[p + "ffn.fc1.weight"], t[p + "ffn.fc1.bias"] = n(f, d), n(f, std=0.01)
        t[p + "ffn.fc2.weight"], t[p + "ffn.fc2.bias"] = n(d, f), n(d, std=0.01)
        for k in "12":
            t[p + f"ln{k}.weight"], t[p + f"ln{k}.bias"] = n(d, mean=1.0), n(d)
    path = os.path.join(folder, "model.nfw")
    nfw_writer.write_nfw(path, t, verbose=False)
    cfg = dict(SIZES, n_layers=n_layers, model_name="gpt2", model_version="1.0.0", bos_token_id=50256,
               eos_token_id=50256, pad_token_id=0, layer_norm_eps=1e-5, pre_norm=True, use_rms_norm=False,
               tie_embeddings=True, pos_embedding="learned", activation="gelu", temperature=0.8, top_p=0.9,
               top_k=50, max_new_tokens=256)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh, indent=1)
    return path


class Params(ctypes.Structure):     # VlrfModelParams, include/api/vlrf.h:52-84
    _fields_ = [(k, ctypes.c_int32) for k in ("vocab_size", "d_model", "d_ff", "n_heads", "n_kv_heads", "n_layers",
                                              "max_seq_len", "bos_token_id", "eos_token_id", "pad_token_id")] + \
               [("temperature", ctypes.c_float), ("top_p", ctypes.c_float), ("top_k", ctypes.c_int32),
                ("max_new_tokens", ctypes.c_int32), ("use_sampling", ctypes.c_int32), ("kv_cache_dtype", ctypes.c_int32),
                ("repetition_penalty", ctypes.c_float), ("frequency_penalty", ctypes.c_float),
                ("presence_penalty", ctypes.c_float), ("no_repeat_ngram_size", ctypes.c_int32),
                ("_reserved", ctypes.c_int32 * 11)]


CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int32, ctypes.c_char_p)


def bind(lib_path: str):
    lib = ctypes.CDLL(lib_path)
    lib.vlrf_create_model.restype = ctypes.c_void_p
    lib.vlrf_load_weights.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p]
    lib.vlrf_get_params.argtypes = [ctypes.c_void_p, ctypes.POINTER(Params)]
    lib.vlrf_set_generation_params.argtypes = [ctypes.c_void_p, ctypes.POINTER(Params)]
    lib.vlrf_generate_ids.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32,
                                      ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32), ctypes.c_int32,
                                      CALLBACK, ctypes.c_void_p]
    lib.vlrf_get_logits.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32,
                                    ctypes.POINTER(ctypes.c_float)]
    lib.vlrf_reset_context.argtypes = [ctypes.c_void_p]
    lib.vlrf_free_model.argtypes = [ctypes.c_void_p]
    lib.vlrf_free_model.restype = None
    lib.vlrf_status_str.restype = ctypes.c_char_p
    lib.vlrf_version.restype = ctypes.c_char_p
    return lib


def check(lib, status: int, what: str) -> None:
    if status != 0:
        raise Unavailable(f"the reference's {what} returned '{lib.vlrf_status_str(status).decode()}'")


def run(steps: int, warmup: int, batch: int, budget_s: float, n_layers: int) -> dict:
    import numpy as np
    ensure_sources()
    lib = bind(ensure_library())
    with tempfile.TemporaryDirectory(prefix="vlrf_reference_arm_") as tmp:
        nfw = write_checkpoint(tmp, n_layers)
        model = lib.vlrf_create_model()
        check(lib, lib.vlrf_load_weights(model, nfw.encode(), None), "vlrf_load_weights")
    try:
        p = Params()
        check(lib, lib.vlrf_get_params(model, ctypes.byref(p)), "vlrf_get_params")
        if p.max_seq_len < SIZES["max_seq_len"]:
            raise Unavailable(f"the reference capped its context to {p.max_seq_len} for want of memory")
        p.use_sampling = 0      # greedy, as the other arm decodes
        p.repetition_penalty = 1.0
        check(lib, lib.vlrf_set_generation_params(model, ctypes.byref(p)), "vlrf_set_generation_params")
        rs = np.random.RandomState(1)
        prompts = rs.randint(0, SIZES["vocab_size"] - 1, size=(batch, PROMPT_LEN)).astype(np.int32)   # never the eos id
        stamps: list = []

        def on_token(_user, _tok, _text):
            stamps.append(time.perf_counter())
            return 1

        cb = CALLBACK(on_token)
        out = (ctypes.c_int32 * (PROMPT_LEN + warmup + steps + 8))()
        decode_s, decode_tokens, sequences = 0.0, 0, 0
        t_start = time.perf_counter()
        for b in range(batch):
            stamps.clear()
            n = ctypes.c_int32(len(out))
            check(lib, lib.vlrf_reset_context(model), "vlrf_reset_context")
            ids = prompts[b].ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
            check(lib, lib.vlrf_generate_ids(model, ids, PROMPT_LEN, out, ctypes.byref(n), warmup + steps, cb, None),
                  "vlrf_generate_ids")
            if len(stamps) < warmup + steps:
                raise Unavailable(f"the reference stopped after {len(stamps)} of {warmup + steps} tokens")
            decode_s += stamps[warmup + steps - 1] - stamps[warmup - 1]     # K steps after W untimed ones
            decode_tokens += steps
            sequences += 1
            if time.perf_counter() - t_start > budget_s:
                break
        # the prompt figure: 2 x 1,024 tokens as two calls of 1,024 (one sequence at a time)
        logits = (ctypes.c_float * SIZES["vocab_size"])()
        long_prompt = rs.randint(0, SIZES["vocab_size"], size=1024).astype(np.int32)
        lp = long_prompt.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
        t0 = time.perf_counter()
        for _ in range(2):
            check(lib, lib.vlrf_get_logits(model, lp, 1024, logits), "vlrf_get_logits")
        prefill_s = time.perf_counter() - t0
        version = lib.vlrf_version().decode()
    finally:
        lib.vlrf_free_model(model)
    tok_s = decode_tokens / decode_s
    return dict(tok_s=tok_s, ms_per_step=1e3 * decode_s / decode_tokens, sequences=sequences,
                prefill_tok_s=2048 / prefill_s, prefill_ms=1e3 * prefill_s, version=version)


def line(steps: int, warmup: int, batch: int, budget_s: float = 60.0, n_layers: int = SIZES["n_layers"]) -> dict:
    try:
        r = run(steps, warmup, batch, budget_s, n_layers)
    except Unavailable as e:
        return {"impl": "reference", "unavailable": str(e)}
    return {
        "metric": "decode tokens/s (GPT-2 small sizes, batch 8, context 1024)", "value": round(r["tok_s"], 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(r["ms_per_step"], 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic (seeded random token ids, random weights)", "impl": "reference",
        "config": {"model": "gpt2", "n_layer": n_layers, "n_layer_of_config": SIZES["n_layers"], "n_embd": SIZES["d_model"],
                   "n_head": SIZES["n_heads"], "n_inner": SIZES["d_ff"], "vocab_size": SIZES["vocab_size"],
                   "n_positions": SIZES["max_seq_len"], "global_batch": batch, "prompt_len": PROMPT_LEN,
                   "same_config": False, "device": f"host CPU, {os.cpu_count()} cores, float32",
                   "batching": f"none in the reference: {r['sequences']} of {batch} sequences one after another",
                   "library": f"libvlrf.so {r['version']} built from baseline/_ref by its CMakeLists.txt (AVX2)",
                   "api": "vlrf_load_weights, vlrf_generate_ids, vlrf_get_logits"},
        "e2e": {"value": round(r["tok_s"], 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the same call: vlrf_generate_ids takes and returns host token ids"},
        "gpu_launches": 0,
        "prefill": {"value": round(r["prefill_tok_s"], 1), "tokens": 2048, "ms": round(r["prefill_ms"], 1), "frac": None},
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--budget-s", type=float, default=60.0, help="stop starting new sequences after this long")
    ap.add_argument("--layers", type=int, default=SIZES["n_layers"])
    args = ap.parse_args()
    print(json.dumps(line(args.steps, max(3, args.warmup), args.batch, args.budget_s, args.layers)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
