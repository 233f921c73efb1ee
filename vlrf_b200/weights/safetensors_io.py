"""Reading and writing `model.safetensors` with nothing but the file format.

Layout: u64 little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}`, then the raw
little-endian data.  The reference's numpy reader shows the same layout and the
bf16 convention, bf16 being the high 16 bits of a float32
(tools/converter/convert_safetensors.py:54-88).  The file is memory-mapped and
each tensor is a view into the map until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import numpy as np
import torch


class WeightError(ValueError):
    """A checkpoint that cannot be used: unreadable, malformed, or not matching
    the tensors that the architecture expects."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """All tensors of a file by name, as CPU tensors in the dtype they are stored in."""
    path = Path(path)
    try:
        f = open(path, "rb")
    except OSError as exc:
        raise WeightError(f"cannot open {path}: {exc}") from exc
    with f:
        size = path.stat().st_size
        if size < 8:
            raise WeightError(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightError(f"{path}: header length {hlen} does not fit a file of {size} bytes")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightError(f"{path}: header is not valid JSON: {exc}") from exc
        if not isinstance(header, dict):
            raise WeightError(f"{path}: header must be a JSON object")
        base = 8 + hlen
        data_len = size - base
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
    out: dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dt, shape, (b, e) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError) as exc:
            raise WeightError(f"{path}: entry '{name}' is malformed: {meta!r}") from exc
        if dt not in _DTYPES:
            raise WeightError(f"{path}: tensor '{name}' has unsupported dtype {dt}; supported: "
                              + ", ".join(sorted(_DTYPES)))
        tdtype, isz = _DTYPES[dt]
        numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if not (0 <= b <= e <= data_len) or e - b != numel * isz:
            raise WeightError(
                f"{path}: tensor '{name}' {dt}{list(shape)} needs {numel * isz} bytes but its offsets "
                f"[{b}, {e}) give {e - b} within {data_len} bytes of data")
        if numel == 0:
            out[name] = torch.empty(shape, dtype=tdtype)
            continue
        arr = np.frombuffer(mm, dtype=np.uint8, count=e - b, offset=base + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nothing writes through the view
            t = torch.from_numpy(arr)
        out[name] = t.view(tdtype).reshape(shape)  # shape () gives a 0-d tensor
    return out


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write tensors in the dtype they have (float32, bfloat16, float16, int32, int64)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * ((8 - len(hbytes) % 8) % 8)  # keep the data 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        for raw in blobs:
            f.write(raw)
