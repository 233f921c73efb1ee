"""Named configurations kept as data: each preset is a config.json-shaped file
beside this module, read through the same path as a model folder's config.json."""
from __future__ import annotations

import json
from pathlib import Path

_HERE = Path(__file__).parent


def preset_names() -> list[str]:
    return sorted(p.stem for p in _HERE.glob("*.json"))


def load_preset(name: str) -> dict:
    path = _HERE / f"{name}.json"
    if not path.exists():
        raise KeyError(f"unknown preset '{name}'; known: {', '.join(preset_names())}")
    return json.loads(path.read_text())
