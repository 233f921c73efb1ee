"""One registry from an architecture's name to what builds it.

An entry holds the configuration class that reads the architecture's
config.json, the function that lists the tensors a checkpoint must hold, the
function that draws random weights, and the function that assembles the model
from parts.  `model_type` in config.json selects the entry everywhere in the
framework: loading, random-weights mode, trace replay, the command line.

The reference has no such table: it guesses the architecture from names in its
Python converters only (tools/converter/convert.py:84-94,
tools/converter/convert_safetensors.py:411).
"""
from __future__ import annotations

import dataclasses
from typing import Callable

from .config.base import ConfigError, ModelConfig


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    #: config -> list[TensorSpec]: every tensor a checkpoint must hold, by name
    weight_spec: Callable
    #: (config, torch.Generator) -> dict name -> float32 tensor, for random-weights mode
    random_weights: Callable
    #: (config, CheckedWeights, BuildOptions) -> engine.model.DecoderModel
    build: Callable
    #: spellings that a checkpoint may put in front of every tensor name of `weight_spec` ("" = none)
    prefixes: tuple = ("",)
    #: config -> fnmatch patterns of tensors that a checkpoint may carry but no computation reads (buffers of
    #: the training code, a head that is tied to the embedding): present or absent, they are no error
    ignored_tensors: Callable = lambda cfg: ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def _load_builtin() -> None:
    """The architectures that ship with the package register themselves when their module is imported."""
    import importlib
    importlib.import_module("vlrf_b200.models")


def architecture_names() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"no architecture registered under '{name}'; registered: "
            + (", ".join(architecture_names()) or "(none)")) from None


def architecture_of(config_dict: dict) -> Architecture:
    """The entry that a config.json's `model_type` names."""
    mt = config_dict.get("model_type")
    if not isinstance(mt, str) or not mt:
        raise ConfigError("config.json has no 'model_type'; registered: " + ", ".join(architecture_names()))
    return get_architecture(mt)


def parse_config(config_dict: dict) -> tuple[Architecture, ModelConfig]:
    arch = architecture_of(config_dict)
    return arch, arch.config_cls.from_dict(config_dict)
