from .engine_config import EngineConfig
from .model_config import ConfigError, read_config_json
from .registry import (
    Architecture,
    architecture_of,
    get_architecture,
    known_architectures,
    load_model_config,
    register_architecture,
    unregister_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "architecture_of",
    "get_architecture",
    "known_architectures",
    "load_model_config",
    "read_config_json",
    "register_architecture",
    "unregister_architecture",
]
