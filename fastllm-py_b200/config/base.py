"""Typed reading of config.json keys.

fastllm-py reads config.json through `_get(cfg, *aliases, default=...)`, which
takes the first alias that is present and not null (fastllm_py/config.py:70-74),
and merges a nested `text_config` over the top level (config.py:82-85).  The
same two rules live here, plus what the reference lacks: a type check on every
value and one error type that names the key.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

_REQUIRED = object()


class ConfigError(ValueError):
    """A config.json that this engine cannot run; the message names the key."""


def read_raw_config(model_path) -> dict:
    """The config.json of a model folder with `text_config` merged over it."""
    path = Path(model_path) / "config.json"
    if not path.exists():
        raise ConfigError(f"no config.json in {model_path}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    if isinstance(raw.get("text_config"), dict):
        merged = dict(raw)
        merged.update(raw["text_config"])
        raw = merged
    return raw


class KeyReader:
    """Reads typed values out of a raw config dict and remembers what it read."""

    def __init__(self, raw: dict):
        self.raw = raw

    def _find(self, names):
        for n in names:
            if n in self.raw and self.raw[n] is not None:
                return n, self.raw[n]
        return None, None

    def integer(self, *names, default: Any = _REQUIRED, minimum: int | None = 1) -> int:
        key, v = self._find(names)
        if key is None:
            if default is _REQUIRED:
                raise ConfigError(f"config.json lacks {' / '.join(names)}")
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"config.json: {key} must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"config.json: {key} must be >= {minimum}, got {v}")
        return v

    def number(self, *names, default: Any = _REQUIRED, positive: bool = True) -> float:
        key, v = self._find(names)
        if key is None:
            if default is _REQUIRED:
                raise ConfigError(f"config.json lacks {' / '.join(names)}")
            return float(default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {key} must be a number, got {v!r}")
        if positive and not v > 0:
            raise ConfigError(f"config.json: {key} must be > 0, got {v}")
        return float(v)

    def boolean(self, *names, default: bool = False) -> bool:
        key, v = self._find(names)
        if key is None:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: {key} must be true or false, got {v!r}")
        return v

    def string(self, *names, default: Any = _REQUIRED) -> str:
        key, v = self._find(names)
        if key is None:
            if default is _REQUIRED:
                raise ConfigError(f"config.json lacks {' / '.join(names)}")
            return default
        if not isinstance(v, str):
            raise ConfigError(f"config.json: {key} must be a string, got {v!r}")
        return v

    def mapping(self, *names) -> dict | None:
        key, v = self._find(names)
        if key is None:
            return None
        if not isinstance(v, dict):
            raise ConfigError(f"config.json: {key} must be an object, got {v!r}")
        return v
