from .base import ConfigError, load_config_json, read_key
from .llama4 import Llama4Config, RopeScaling
from .presets import PRESETS, preset
from .registry import Architecture, known_architectures, register_architecture, resolve, unregister_architecture

__all__ = [
    "Architecture", "ConfigError", "Llama4Config", "PRESETS", "RopeScaling", "known_architectures",
    "load_config_json", "preset", "read_key", "register_architecture", "resolve", "unregister_architecture",
]
