"""From a model folder to a model on the device."""
from __future__ import annotations

import time

import torch

from .. import log
from ..weights.model_dir import open_model_dir
from .model import BuildOptions, DecoderModel

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}'; choose bfloat16 or float32") from None


def load_model(model_dir, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Read config.json, pick the architecture it names, check model.safetensors against that
    architecture's tensor list and assemble the model on the device."""
    import vlrf_b200.models  # noqa: F401  (registers the architectures)
    arch, cfg, weights = open_model_dir(model_dir)
    options = BuildOptions(dtype=parse_dtype(dtype), device=torch.device(device))
    if options.device.type != "cuda" or not torch.cuda.is_available():
        from ..csrc import KernelError
        raise KernelError(f"cannot put a model on '{device}': the engine's kernels are CUDA code for sm_100a and there "
                          f"is no other execution path (CUDA available: {torch.cuda.is_available()})")
    started = time.perf_counter()
    model = arch.build(cfg, weights, options)
    log.info(f"{model_dir}: {arch.name}, {len(model.layers)} layers, width {model.width}, vocabulary {model.vocab_size}, "
             f"{model.weight_bytes() / 2**20:.1f} MiB of weights as {options.dtype} on {options.device} "
             f"in {time.perf_counter() - started:.2f} s")
    kinds = {}
    for i, name, k in model.describe_kernels():
        kinds.setdefault((name, k["prompt"], k["decode"]), []).append(i)
    for (name, prompt, decode), layers in kinds.items():
        say = log.warn if options.dtype == torch.bfloat16 and "CUDA cores" in (prompt, decode) else log.info
        say(f"layers {layers[0]}…{layers[-1]} ({name}): prompt attention on {prompt}, decode attention on {decode}"
            + (" (no tensor-core kernel takes this head size)" if say is log.warn else ""))
    return model
