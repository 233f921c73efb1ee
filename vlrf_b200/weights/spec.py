"""What a checkpoint must hold, and the one check that compares a file with it.

An architecture lists `TensorSpec`s by tensor name.  `check_tensors` compares
the names and shapes found in a file with that list and raises ONE error that
names every missing tensor, every unexpected tensor and every wrong shape, so a
bad checkpoint is diagnosed in one go.  (The reference stops at the first
missing name: include/model/weights.hpp:152-165.)
"""
from __future__ import annotations

import dataclasses
import fnmatch

import torch

from .safetensors_io import WeightError


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    #: "matrix": operand of a matrix product (bfloat16 in the bfloat16 engine);
    #: "vector": bias / norm parameter (always computed with in 32-bit);
    #: "table": integer table (kept int32)
    kind: str = "matrix"
    optional: bool = False


@dataclasses.dataclass
class CheckedWeights:
    """Tensors that passed `check_tensors`, by the spec's (prefix-free) names."""
    tensors: dict

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def __contains__(self, name: str) -> bool:
        return name in self.tensors


def check_tensors(found: dict, specs: list, *, prefixes: tuple = ("",), ignore: tuple = (),
                  source: str = "checkpoint") -> CheckedWeights:
    """Match `found` (name -> tensor) against `specs`.

    prefixes -- accepted spellings in front of a spec's name (e.g. "transformer.")
    ignore   -- fnmatch patterns of tensors that may be present but are not used
                (mask buffers and the like)
    """
    used = set()
    matched: dict[str, torch.Tensor] = {}
    missing, wrong = [], []
    for spec in specs:
        hit = None
        for p in prefixes:
            if p + spec.name in found:
                hit = p + spec.name
                break
        if hit is None:
            if not spec.optional:
                missing.append(f"{spec.name} {list(spec.shape)}")
            continue
        used.add(hit)
        t = found[hit]
        if tuple(t.shape) != tuple(spec.shape):
            wrong.append(f"{hit}: expected {list(spec.shape)}, found {list(t.shape)}")
            continue
        if spec.kind == "table" and t.is_floating_point():
            wrong.append(f"{hit}: expected an integer table, found {t.dtype}")
            continue
        if spec.kind != "table" and not t.is_floating_point():
            wrong.append(f"{hit}: expected floating point, found {t.dtype}")
            continue
        matched[spec.name] = t
    unexpected = []
    for name in found:
        if name in used:
            continue
        if any(fnmatch.fnmatchcase(name, pat) for pat in ignore):
            continue
        unexpected.append(f"{name} {list(found[name].shape)}")
    if missing or wrong or unexpected:
        lines = [f"{source} does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + "; ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + "; ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))
    return CheckedWeights(matched)


def place(t: torch.Tensor, kind: str, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """Move one checked tensor to the device in the dtype its kind computes in.

    bfloat16 engine: matrices are bfloat16 (a matrix stored in bfloat16 stays as
    stored; one stored wider is rounded once, here); vectors are float32 (a
    vector stored in 32-bit stays so; bfloat16 widens exactly).  float32 engine:
    everything float32 (bfloat16 widens exactly).  Tables are int32.
    """
    if kind == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    if kind == "vector" or compute_dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32).contiguous()
    return t.to(device=device, dtype=torch.bfloat16).contiguous()
