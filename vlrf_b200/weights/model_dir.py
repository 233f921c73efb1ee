"""A model folder: config.json + model.safetensors.

`open_model_dir` reads both and checks the tensors against the list that the
architecture named by config.json gives; `write_random_model` makes such a
folder from a configuration and a seed.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.base import ModelConfig, read_config_json
from ..registry import Architecture, parse_config
from .safetensors_io import WeightError, read_safetensors, write_safetensors
from .spec import CheckedWeights, check_tensors


def open_model_dir(model_dir) -> tuple[Architecture, ModelConfig, CheckedWeights]:
    model_dir = Path(model_dir)
    arch, cfg = parse_config(read_config_json(model_dir))
    st = model_dir / "model.safetensors"
    if not st.exists():
        raise WeightError(f"{model_dir} has no model.safetensors")
    found = read_safetensors(st)
    specs = arch.weight_spec(cfg)
    # which prefixes a checkpoint may carry and which of its tensors nothing reads is the architecture's to say
    checked = check_tensors(found, specs, prefixes=tuple(arch.prefixes), ignore=tuple(arch.ignored_tensors(cfg)),
                            source=str(st))
    return arch, cfg, checked


def write_random_model(config: dict | ModelConfig, seed: int, out_dir, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Random-weights mode: write `out_dir/config.json` and `out_dir/model.safetensors`
    for the architecture that the configuration names.  Floating tensors are
    stored in `dtype`; the draw is made in float32 from `seed` alone."""
    cfg_dict = config.to_dict() if isinstance(config, ModelConfig) else dict(config)
    arch, cfg = parse_config(cfg_dict)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    tensors = arch.random_weights(cfg, gen)
    specs = {s.name: s for s in arch.weight_spec(cfg)}
    stored = {}
    for name, t in tensors.items():
        if name not in specs:
            raise WeightError(f"random weights produced '{name}', which the architecture does not list")
        stored[name] = t.to(dtype) if t.is_floating_point() else t.to(torch.int32)
    check_tensors(stored, list(specs.values()), source="random weights")
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(cfg_dict, indent=2) + "\n")
    write_safetensors(out_dir / "model.safetensors", stored, metadata={"format": "pt", "seed": seed})
    return out_dir
