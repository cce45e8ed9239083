from .base import ConfigError, read_raw_config
from .engine import EngineConfig, canonical_dtype
from .llama import LinearRopeScaling, LlamaConfig
from .registry import (Architecture, architecture_names, architecture_of, load_config,
                       register_architecture)

__all__ = [
    "ConfigError", "read_raw_config", "EngineConfig", "canonical_dtype", "LinearRopeScaling",
    "LlamaConfig", "Architecture", "architecture_names", "architecture_of", "load_config",
    "register_architecture",
]
