"""A B200-native inference engine for the Llama / DeepSeek-LLM dense decoder.

Public names follow fastllm-py's (`from fastllm_py import Model, load_config`,
fastllm_py/__init__.py:1-4)."""
from . import architectures  # noqa: F401
from .api import Model
from .config import ConfigError, EngineConfig, LlamaConfig, load_config, register_architecture
from .engine import Engine, Scheduler, StepEntry
from .parts import register_part
from .sampling import SamplingParams
from .weights import WeightError, write_model_folder

__all__ = ["Model", "ConfigError", "EngineConfig", "LlamaConfig", "load_config",
           "register_architecture", "Engine", "Scheduler", "StepEntry", "register_part",
           "SamplingParams", "WeightError", "write_model_folder"]
