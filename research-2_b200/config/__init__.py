from .registry import (
    Architecture,
    ConfigError,
    architecture,
    architecture_of,
    known_architectures,
    load_config,
    read_config_json,
    register_architecture,
    unregister_architecture,
)
from .engine_options import EngineOptions
from .gpt2 import GPT2Config

__all__ = [
    "Architecture", "ConfigError", "EngineOptions", "GPT2Config", "architecture", "architecture_of",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
    "unregister_architecture",
]
