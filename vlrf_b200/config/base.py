"""Typed model configurations read from an architecture's own config.json keys.

A configuration class lists its keys as dataclass fields whose metadata says
how config.json spells them and which Python type they must have.  Nothing
here knows a particular architecture; `vlrf_b200.registry` maps the
`model_type` of a config.json to the class that reads it.

The reference reads a converter-written dialect with a substring search
(src/api/vlrf_api.cpp:582-681) and keeps generation defaults in the same struct
(include/model/config.hpp:32-124); here the Hugging Face keys are read directly
with a real JSON parser, and sampling options live with the generation loop.
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the named architecture."""


_MISSING = object()


def key(json_key: str | None = None, *, default: Any = _MISSING, nullable: bool = False):
    """Declare a configuration field.

    json_key  -- spelling in config.json (defaults to the field name)
    default   -- value when the key is absent; without one the key is required
    nullable  -- whether JSON null is accepted (stored as None)
    """
    md = {"json_key": json_key, "nullable": nullable, "required": default is _MISSING}
    if default is _MISSING:
        return dataclasses.field(metadata=md)
    return dataclasses.field(default=default, metadata=md)


def _check_type(name: str, value: Any, annotation: str, nullable: bool) -> Any:
    if value is None:
        if nullable:
            return None
        raise ConfigError(f"config key '{name}' must not be null")
    base = annotation.replace("| None", "").replace("Optional[", "").replace("]", "").strip()
    if base.startswith("<class '"):
        base = base[len("<class '"):-2]
    if base == "int":
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"config key '{name}' must be an integer, got {value!r}")
        return value
    if base == "float":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key '{name}' must be a number, got {value!r}")
        return float(value)
    if base == "bool":
        if not isinstance(value, bool):
            raise ConfigError(f"config key '{name}' must be true or false, got {value!r}")
        return value
    if base == "str":
        if not isinstance(value, str):
            raise ConfigError(f"config key '{name}' must be a string, got {value!r}")
        return value
    return value


@dataclasses.dataclass
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses add fields with `key(...)`, set `model_type`, and override
    `validate()` for the relations between their sizes.
    """

    model_type = ""  # class attribute: the config.json "model_type" this class reads

    @classmethod
    def from_dict(cls, data: dict) -> "ModelConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        kwargs = {}
        missing = []
        for f in dataclasses.fields(cls):
            md = f.metadata
            if "json_key" not in md:
                continue
            jk = md["json_key"] or f.name
            if jk in data:
                kwargs[f.name] = _check_type(jk, data[jk], str(f.type), md["nullable"])
            elif md["required"]:
                missing.append(jk)
        if missing:
            raise ConfigError(
                f"config.json of model_type '{cls.model_type}' lacks required key(s): " + ", ".join(missing))
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path) -> "ModelConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict:
        out = {"model_type": self.model_type}
        for f in dataclasses.fields(self):
            md = f.metadata
            if "json_key" in md:
                out[md["json_key"] or f.name] = getattr(self, f.name)
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    @staticmethod
    def _positive(name: str, value: int) -> None:
        if value <= 0:
            raise ConfigError(f"config key '{name}' must be positive, got {value}")


def read_config_json(path) -> dict:
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    try:
        text = path.read_text()
    except OSError as exc:
        raise ConfigError(f"cannot read {path}: {exc}") from exc
    try:
        data = json.loads(text)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data
