"""The command line, with the commands, option names and defaults of the reference's CLI where it has
them (tools/vlrf_cli.cpp:93-121, usage :123-170):

    python -m vlrf_b200.cli run  --model DIR (--prompt "text" | --prompt-ids 1,2,3 | --prompts-file F)
                                 [--tokens N] [--ctx N] [--temp F] [--seed N] [--greedy]
                                 [--repeat-penalty F] [--freq-penalty F] [--presence-penalty F]
                                 [--no-repeat-ngram N] [--top-k N] [--top-p F] [--stop-id N ...]
                                 [--dtype bfloat16|float32]
    python -m vlrf_b200.cli info --model DIR
    python -m vlrf_b200.cli init --config PRESET|config.json --out DIR [--seed N]

`--model` is a folder with config.json and model.safetensors (the reference takes its own .nfw file).
Without a tokenizer, `--prompt "text"` is encoded like the reference does without one: byte + 4, capped
at the vocabulary (src/api/vlrf_api.cpp:373-381); token ids are printed, since there is nothing to decode
them with.  `--stop` (stop strings) needs a tokenizer and is not offered; `--stop-id` stops at token ids.
`--ctx N` sizes the cache in tokens (vlrf_set_ctx there).  `--temp` is applied here (the reference's CLI
parses it and drops it).  `init` writes a random-weights model folder (disabled there).  `--backend` and
`--kv-cache` do not exist: there is one backend and the cache has the engine's dtype.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def _add_run_options(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--prompts-file", default=None, help="one comma- or space-separated id list per line: a batch")
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=0, help="tokens the cache holds; 0 = enough for this call")
    ap.add_argument("--temp", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--freq-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--no-repeat-ngram", type=int, default=0)
    ap.add_argument("--stop-id", type=int, action="append", default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])


def _prompts(args) -> tuple[list, bool]:
    """(prompts, whether they are bytes of --prompt text that still want the cap at the vocabulary)."""
    if args.prompts_file:
        out = []
        for line in Path(args.prompts_file).read_text().splitlines():
            line = line.strip()
            if line:
                out.append([int(t) for t in line.replace(",", " ").split()])
        return out, False
    if args.prompt_ids is not None:
        return [[int(t) for t in args.prompt_ids.replace(",", " ").split()]], False
    if args.prompt is not None:
        return [[b + 4 for b in args.prompt.encode("utf-8")]], True
    raise SystemExit("run: give --prompt, --prompt-ids or --prompts-file")


def cmd_run(args) -> int:
    from . import Model, SamplingParams
    prompts, from_text = _prompts(args)
    need = sum((len(p) + args.tokens + 63) // 64 * 64 for p in prompts)
    print(f"Loading model from {args.model} ...")
    model = Model.load(args.model, dtype=args.dtype, max_tokens=args.ctx if args.ctx > 0 else need)
    print(model.model_summary())
    if from_text:       # bytes beyond the vocabulary become its last id (src/api/vlrf_api.cpp:373-381)
        prompts = [[min(t, model.decoder.vocab_size - 1) for t in p] for p in prompts]
    params = SamplingParams(
        max_new_tokens=args.tokens, temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
        do_sample=not args.greedy, repetition_penalty=args.repeat_penalty, frequency_penalty=args.freq_penalty,
        presence_penalty=args.presence_penalty, no_repeat_ngram_size=args.no_repeat_ngram, seed=args.seed,
        stop_token_ids=tuple(args.stop_id) if args.stop_id else None)
    t0 = time.time()
    results = model.generate_ids(prompts, params)
    dt = time.time() - t0
    total = 0
    for i, r in enumerate(results):
        print(f"--- Prompt {i} ---\n{' '.join(map(str, r.prompt))}\n--- Output ({r.finish_reason}) ---")
        print(" ".join(map(str, r.new_tokens)))
        total += r.tokens_generated
    ctx = sum(len(r.token_ids) for r in results)
    print(f"\n[{ctx} tokens in context, {total} generated, {dt:.2f} s, {total / max(dt, 1e-9):.1f} tok/s]")
    return 0


def cmd_info(args) -> int:
    import vlrf_b200.models  # noqa: F401
    from .config.base import read_config_json
    from .registry import parse_config
    arch, cfg = parse_config(read_config_json(args.model))
    print(f"architecture: {arch.name}")
    print(json.dumps(cfg.to_dict(), indent=2))
    if hasattr(cfg, "param_count"):
        print(f"parameters: {cfg.param_count():,}")
    return 0


def cmd_init(args) -> int:
    import vlrf_b200.models  # noqa: F401
    from .config import load_preset, preset_names
    from .weights import write_random_model
    if args.config in preset_names():
        cfg = load_preset(args.config)
    else:
        try:
            cfg = json.loads(Path(args.config).read_text())
        except (OSError, ValueError) as exc:
            from .config.base import ConfigError
            raise ConfigError(f"--config {args.config}: neither a preset ({', '.join(sorted(preset_names()))}) "
                              f"nor a readable config.json ({exc})") from exc
    out = write_random_model(cfg, args.seed, args.out)
    print(f"wrote {out}/config.json and {out}/model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="vlrf_b200", description="GPT-2 inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    _add_run_options(sub.add_parser("run", help="generate from prompts"))
    sub.add_parser("info", help="print the model's configuration").add_argument("--model", required=True)
    pi = sub.add_parser("init", help="write a model folder with random weights")
    pi.add_argument("--config", required=True, help="a preset name or a config.json")
    pi.add_argument("--out", required=True)
    pi.add_argument("--seed", type=int, default=1234)
    args = ap.parse_args(argv)
    from .cache import CacheError
    from .config.base import ConfigError
    from .csrc import KernelError
    from .engine.generate import GenerationError
    from .engine.step import StepError
    from .weights.safetensors_io import WeightError
    try:
        return {"run": cmd_run, "info": cmd_info, "init": cmd_init}[args.command](args)
    except (ConfigError, WeightError, GenerationError, StepError, CacheError, KernelError) as exc:
        # what the library itself refuses is a message and a status, as with the reference's CLI; anything else is a fault
        # of the program and keeps its traceback
        print(f"vlrf_b200 {args.command}: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
