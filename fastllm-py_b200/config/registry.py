"""The one registry from an architecture's name to its configuration and model.

fastllm-py has no registry: one generic forward serves every family and finds
features by looking at which tensor names exist (fastllm_py/model.py:1-5).
Here `config.json["architectures"][0]` (or `model_type`, for folders that lack
it) picks an entry, and an entry is two things: the typed configuration class
and the function that turns a configuration into a ModelPlan, the description
of the model in terms of parts.  Adding an architecture is one call of
`register_architecture`; nothing else in the package names an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, read_raw_config


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type          # has classmethod from_hf(raw: dict) and method to_hf() -> dict
    make_plan: Callable         # (config, tensor_names: set[str] | None) -> ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(name: str, config_class: type, make_plan: Callable,
                          model_types: tuple[str, ...] = ()) -> None:
    """Make `name` (as in config.json's `architectures`) loadable.

    `model_types` are values of config.json's `model_type` that select this
    architecture when `architectures` is absent."""
    _ARCHITECTURES[name] = Architecture(name, config_class, make_plan)
    for t in model_types:
        _MODEL_TYPES[t] = name


def architecture_names() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: dict) -> Architecture:
    names = raw.get("architectures")
    name = None
    if isinstance(names, list) and names:
        name = names[0]
    elif isinstance(raw.get("model_type"), str):
        name = _MODEL_TYPES.get(raw["model_type"])
        if name is None:
            raise ConfigError(
                f"config.json has no 'architectures' and model_type {raw['model_type']!r} "
                f"is not registered (known: {sorted(_MODEL_TYPES)})")
    if name is None:
        raise ConfigError("config.json has neither 'architectures' nor 'model_type'")
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered (known: {architecture_names()})")
    return _ARCHITECTURES[name]


def load_config(model_path):
    """(architecture entry, typed configuration) of a model folder."""
    raw = read_raw_config(model_path)
    arch = architecture_of(raw)
    return arch, arch.config_class.from_hf(raw)
