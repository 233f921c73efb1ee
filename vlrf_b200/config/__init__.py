from .base import ConfigError, ModelConfig, key, read_config_json
from .gpt2 import GPT2Config
from .presets import load_preset, preset_names

__all__ = ["ConfigError", "ModelConfig", "key", "read_config_json", "GPT2Config",
           "load_preset", "preset_names"]
