"""Trace replay: feed given token ids through a model step by step and write the logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` gives for each request its next tokens and the places among them whose logits are wanted;
`end` lists requests that are finished after the step, whose slot and blocks go back to the cache.  For a
step that wants something, `OUT/<step>.f32` holds the wanted logits in the order of the entries and of
`want`, little-endian float32 [wanted, vocab].  After every step the line `done <step>` is printed and
flushed.  Nothing is sampled.  The model, the step function, the cache and the kernels are the ones that
generation uses (`vlrf_b200.engine`); this module only parses lines and writes files.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time, each rounded up to a multiple of 64")
    args = ap.parse_args(argv)

    print("[trace_run] loading (the first call in a fresh checkout compiles the CUDA kernels)",
          file=sys.stderr, flush=True)
    import numpy as np
    import torch  # noqa: F401
    from .engine.loading import load_model
    from .engine.step import Engine, StepEntry

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, args.dtype, "cuda:0")
    engine = Engine(model, max_tokens=args.max_tokens)
    print("[trace_run] ready", file=sys.stderr, flush=True)

    slot_of: dict = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries = []
        for e in msg.get("entries", []):
            rid = e["id"]
            if rid not in slot_of:
                slot_of[rid] = engine.start_sequence()
            entries.append(StepEntry(slot_of[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = out_dir / f"{step}.f32.tmp"
                np.ascontiguousarray(arr).tofile(tmp)
                tmp.replace(out_dir / f"{step}.f32")
            engine.check_device_errors()
        for rid in msg.get("end", []):
            if rid in slot_of:
                engine.end_sequence(slot_of.pop(rid))
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
