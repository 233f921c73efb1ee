#!/usr/bin/env python3
"""Decode and prefill throughput of the GPT-2 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--preset gpt2] [--batch 8]

A step is one decode step of the whole batch: every sequence goes on by one token.  The default run has
the layer sizes of the GPT-2 small configuration with random weights (seeded, synthetic token ids), a
batch of 8 and a context of 1,024: the sequences start from 512-token prompts and decode to 1,024 (16 warm-up
steps, then the 496 timed ones).
One JSON line is printed:

  value      decoded tokens a second, K steps timed on the device with CUDA events after W warm-up steps;
             the sampled tokens feed the next step on the device
  e2e        the same through the Python entry point (`Model.generate_ids`): every step copies its input
             tokens from pinned host memory to the device and reads the sampled tokens back
  prefill    one step of 2 x 1,024 prompt tokens: tokens a second, and its flops / time / the bf16 peak; the
             engine replays a captured graph for a step of a shape it has run before, which the timed
             repetitions are; `ms_new_shape` is the same step launched kernel by kernel from the host, as
             the first step of a new shape is
  roofline   decode: bytes the step has to read (every weight it uses once, the cache of the live
             sequences) / its time, against the HBM copy peak
  points     decode tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the fallback
figures 6.65 TB/s and 1.59 PFLOP/s.  The working set of a step (weights + cache, > 400 MB) is larger than
the 126 MB L2, so no L2 flush is issued between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PROMPT_LEN = 512


def peaks(root: str = ROOT):
    """(HBM copy GB/s, bf16 TFLOP/s of a burst, "measured" | "fallback").  The measured file gives `hbm_gbs` and
    `bf16_tflops` as numbers (a figure wrapped as {"value": x} is read too); anything else in it, or a file that
    does not parse, leaves the fallback figure for that peak."""
    path = os.path.join(root, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"

    def number(v):
        if isinstance(v, dict):
            v = v.get("value")
        if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
            return float(v)
        return None

    try:
        with open(path) as f:
            p = json.load(f)
    except (OSError, ValueError):
        return hbm, tf, src
    if isinstance(p, dict):
        got_hbm, got_tf = number(p.get("hbm_gbs")), number(p.get("bf16_tflops"))
        if got_hbm is not None:
            hbm, src = got_hbm, "measured"
        if got_tf is not None:
            tf, src = got_tf, "measured"
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: through NVML every few
    milliseconds (read-only queries), or with nvidia-smi if the NVML module is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, period_s: float = 0.005):
        self.samples, self.proc, self.thread = [], None, None
        self.period_s, self.stop = period_s, threading.Event()

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:  # noqa: BLE001 - no NVML: ask nvidia-smi instead
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self, pynvml, handle):
        reasons_of = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        try:
            mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            while not self.stop.is_set():
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                bits = int(reasons_of(handle))
                flags = ["Active" if bits & self.REASON_BITS[n] else "Not Active"
                         for n in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")]
                self.samples.append(", ".join([str(sm), str(mx)] + flags))
                self.stop.wait(self.period_s)
        except Exception:  # noqa: BLE001 - a failed query ends the sampling, not the benchmark
            pass

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def step_bytes(model, engine, slots) -> int:
    """Bytes a decode step has to read: every weight it uses once (the position table only the rows of
    this step) and the keys and values of the live sequences."""
    cfg = model.config
    w = model.weight_bytes()
    wpe_all = cfg.n_positions * cfg.n_embd * (2 if model.act_dtype.itemsize == 2 else 4)
    wpe_used = len(slots) * cfg.n_embd * (2 if model.act_dtype.itemsize == 2 else 4)
    return w - wpe_all + wpe_used + engine.cache.live_kv_bytes(slots)


def prefill_flops(cfg, lens, n_logit_rows) -> float:
    d, f, L, H = cfg.n_embd, cfg.inner_dim, cfg.n_layer, cfg.n_head
    T = sum(lens)
    gemm = 2.0 * T * (3 * d * d + d * d + 2 * d * f) * L
    attn = sum(4.0 * (d // H) * (s * (s + 1) / 2) * H for s in lens) * L
    head = 2.0 * n_logit_rows * d * cfg.vocab_size
    return gemm + attn + head


def make_model_dir(preset: str, n_layer: int | None, tmp: str) -> str:
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.config import load_preset
    from vlrf_b200.weights import write_random_model
    cfg = load_preset(preset)
    if n_layer is not None:
        cfg["n_layer"] = n_layer
    return str(write_random_model(cfg, 1234, os.path.join(tmp, "model")))


def random_prompts(vocab, batch, length, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g).tolist()


def decode_device(model_dir, batch, steps, warmup, dtype="bfloat16"):
    """K decode steps timed on the device; tokens stay on the device between steps."""
    import torch
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    model = load_model(model_dir, dtype)
    cfg = model.config
    ctx_len = cfg.n_positions
    steps = min(steps, ctx_len - PROMPT_LEN - warmup)
    engine = Engine(model, max_tokens=batch * ctx_len, n_slots=batch)
    prompts = random_prompts(cfg.vocab_size, batch, PROMPT_LEN, 1)
    slots = [engine.start_sequence() for _ in range(batch)]
    out = torch.zeros(batch, dtype=torch.int32, device=model.device)
    for b0 in range(0, batch, 8):      # prompts in steps of 8 sequences
        idx = list(range(b0, min(batch, b0 + 8)))
        logits = engine.step([StepEntry(slots[i], prompts[i], [PROMPT_LEN - 1]) for i in idx])
        ops.sample(logits, len(idx), out[b0:b0 + len(idx)])
    sess = DecodeSession(engine, slots, use_graph=True)
    sess.reserve_ahead(warmup + steps + 1)
    sess.set_tokens(out)
    for _ in range(warmup):
        sess.step_greedy(out)
    torch.cuda.synchronize()
    bytes_first = step_bytes(model, engine, slots)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clk:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            sess.step_greedy(out)        # model + argmax + hand-over to the next step: one replayed graph
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    bytes_last = step_bytes(model, engine, slots)
    engine.check_device_errors()
    launches = steps * sess.kernels_per_step              # the step's kernels, sampling included (replayed)
    return dict(tok_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, steps=steps,
                bytes_per_step=(bytes_first + bytes_last) / 2, clocks=clk.summary(), launches=launches,
                kernels_per_step=sess.kernels_per_step, mean_context=PROMPT_LEN + warmup + steps / 2,
                weight_bytes=model.weight_bytes(), n_layer=cfg.n_layer)


def decode_e2e(model_dir, batch, steps, warmup, dtype="bfloat16"):
    """The same K steps through Model.generate_ids: host tokens in and out at every step."""
    import torch
    from vlrf_b200 import Model, SamplingParams
    model = Model.load(model_dir, dtype=dtype, max_tokens=batch * 1024, n_slots=batch)
    cfg = model.config
    steps = min(steps, cfg.n_positions - PROMPT_LEN - warmup - 2)
    prompts = random_prompts(cfg.vocab_size, batch, PROMPT_LEN, 1)
    marks = {}
    count = [0]

    def on_token(index, tok):
        if index != 0:
            return True
        count[0] += 1                       # token number of request 0 = step number
        if count[0] == warmup + 1:          # prompt step and W decode steps are done
            torch.cuda.synchronize()
            marks["t0"] = time.perf_counter()
            marks["h2d0"], marks["d2h0"] = model.backend.h2d_bytes, model.backend.d2h_bytes
        elif count[0] == warmup + 1 + steps:
            torch.cuda.synchronize()
            marks["t1"] = time.perf_counter()
            marks["h2d1"], marks["d2h1"] = model.backend.h2d_bytes, model.backend.d2h_bytes
        return True

    params = SamplingParams(max_new_tokens=warmup + steps + 2, do_sample=False, stop_token_ids=())
    model.generate_ids(prompts, params, on_token=on_token)
    dt = marks["t1"] - marks["t0"]
    return dict(tok_s=batch * steps / dt, h2d=(marks["h2d1"] - marks["h2d0"]) / steps,
                d2h=(marks["d2h1"] - marks["d2h0"]) / steps, steps=steps)


def prefill_device(model_dir, dtype="bfloat16", reps=5, replay=True):
    """One step of 2 x 1,024 prompt tokens.  replay: the engine replays a captured graph for a step whose shape
    it has seen before (the default); without it every kernel is launched from the host, as for a new shape."""
    import torch
    from vlrf_b200.engine import Engine, StepEntry, load_model
    model = load_model(model_dir, dtype)
    cfg = model.config
    n_seq, length = 2, min(1024, cfg.n_positions)
    engine = Engine(model, max_tokens=n_seq * length, n_slots=n_seq)
    engine.capture_repeated_steps = replay
    import numpy as np
    # host token ids as int32 arrays (a Python list of a thousand ids costs about 30 us to convert, inside the step)
    prompts = [np.asarray(p, dtype=np.int32) for p in random_prompts(cfg.vocab_size, n_seq, length, 2)]
    times = []
    for r in range(reps + 2):
        slots = [engine.start_sequence() for _ in range(n_seq)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepEntry(s, p, [length - 1]) for s, p in zip(slots, prompts)])
        e1.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(e0.elapsed_time(e1))
        for s in slots:
            engine.end_sequence(s)
    engine.check_device_errors()
    ms = statistics.median(times)
    return dict(tokens=n_seq * length, ms=ms, flops=prefill_flops(cfg, [length] * n_seq, n_seq))


def metric_label(preset: str, batch: int, first_context: int, last_context: int) -> str:
    sizes = "GPT-2 small sizes" if preset == "gpt2" else preset
    return f"decode tokens/s ({sizes}, batch {batch}, contexts {first_context} to {last_context})"


def reference_arm(args) -> int:
    """`--impl reference`: the unmodified reference, built from baseline/_ref by its own CMakeLists.txt and driven
    through its C API by baseline/reference_arm.py in a process of its own (nothing of this package is loaded
    there).  It prints the same JSON line, or an `unavailable` line that says why."""
    if args.gpus != 1:
        print(f"bench.py measures one GPU: the reference runs on the host cores (asked for --gpus {args.gpus})")
        return 2
    warmup = max(3, args.warmup)
    steps = min(args.steps, 1024 - PROMPT_LEN - warmup - 2)
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(steps), "--warmup",
           str(warmup), "--batch", str(args.batch)]
    if args.layers is not None:
        cmd += ["--layers", str(args.layers)]
    try:
        done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=900)
        lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
        line = json.loads(lines[-1])
    except (OSError, subprocess.TimeoutExpired, IndexError, ValueError) as e:
        line = {"impl": "reference", "unavailable": f"the reference's harness gave no result ({type(e).__name__})"}
    if "unavailable" not in line:
        line["metric"] = metric_label("gpt2", args.batch, PROMPT_LEN + warmup, PROMPT_LEN + warmup + steps)
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=496, help="decode steps to time (496 after 16 warm-up steps ends at position 1,024)")
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="gpt2")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode or prefill and VLRF_B200_KERNEL_TRACE=1: print where the last step's kernels spent their time")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only and print a short line (for profiling runs); the full line needs 'all'")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from vlrf_b200.config import load_preset
    hbm_gbs, bf16_tflops, peak_src = peaks()
    full_layers = load_preset(args.preset)["n_layer"]
    with tempfile.TemporaryDirectory(prefix="vlrf_b200_bench_") as tmp:
        model_dir = make_model_dir(args.preset, args.layers, tmp)
        if args.only == "decode":
            dec = decode_device(model_dir, args.batch, args.steps, warmup)
            print(json.dumps({"only": "decode", "batch": args.batch, "tok_s": round(dec["tok_s"], 1),
                              "ms_per_step": round(dec["ms_per_step"], 4), "kernels_per_step": dec["kernels_per_step"]}))
            if args.timeline:
                from vlrf_b200 import log
                print(log.timeline_table(log.kernel_timeline(), last=5 * dec["n_layer"]))
            return 0
        if args.only == "prefill":
            pre = prefill_device(model_dir, reps=max(1, args.steps))
            print(json.dumps({"only": "prefill", "tokens": pre["tokens"], "ms": round(pre["ms"], 4)}))
            if args.timeline:
                from vlrf_b200 import log
                print(log.timeline_table(log.kernel_timeline(), last=5 * full_layers if args.layers is None else 5 * args.layers))
            return 0
        dec = decode_device(model_dir, args.batch, args.steps, warmup)
        e2e = decode_e2e(model_dir, args.batch, dec["steps"], warmup)
        pre = prefill_device(model_dir)
        pre_new_shape = prefill_device(model_dir, replay=False)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(decode_device(model_dir, b, min(args.steps, 128), warmup)["tok_s"], 1)
    if not args.skip_points and args.preset == "gpt2" and args.layers is None:
        # the largest size of the family at its full depth, where a step is bound by bytes rather than by latencies
        with tempfile.TemporaryDirectory(prefix="vlrf_b200_bench_") as tmp:
            xl = decode_device(make_model_dir("gpt2-xl", None, tmp), 8, 64, warmup)
        points["xl_decode_b8"] = round(xl["tok_s"], 1)
        points["xl_decode_b8_hbm_frac"] = round(xl["bytes_per_step"] / (xl["ms_per_step"] / 1e3) / 1e9 / hbm_gbs, 4)
    cfg = load_preset(args.preset)
    achieved = dec["bytes_per_step"] / (dec["ms_per_step"] / 1e3) / 1e9
    pre_tflops = pre["flops"] / (pre["ms"] / 1e3) / 1e12
    line = {
        "metric": metric_label(args.preset, args.batch, PROMPT_LEN + warmup, PROMPT_LEN + warmup + dec["steps"]),
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": dec["steps"], "warmup": warmup,
        "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random token ids, random weights)",
        "impl": "ours",
        "config": {
            "model": args.preset, "n_layer": dec["n_layer"], "n_layer_of_config": full_layers,
            "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"] or 4 * cfg["n_embd"],
            "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"], "global_batch": args.batch,
            "seq_len": cfg["n_positions"], "prompt_len": PROMPT_LEN, "mean_context": dec["mean_context"],
            "parallelism": "single GPU", "weights": "bf16 random", "kv_cache": "bf16 paged, 64-token blocks",
            "l2": "working set of a step exceeds L2; no flush", "peaks": peak_src,
            "kernels_per_step": dec["kernels_per_step"],
        },
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(pre["tokens"] / (pre["ms"] / 1e3), 1), "tokens": pre["tokens"],
                    "ms": round(pre["ms"], 4), "frac": round(pre_tflops / bf16_tflops, 4),
                    "ms_new_shape": round(pre_new_shape["ms"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": dec["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
