"""What a mixer asks of the cache manager.

A mixer declares its need; the manager groups equal needs and serves each group
from pages of its own.  fastllm-py has one kind only (every layer keeps all keys
and values, fastllm_py/model.py:76-123), so it has no such notion.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class PagedKV:
    """Keys and values per token: `kv_heads` x `head_dim` each.

    `window` None keeps every token; a number keeps the last `window` tokens
    (the query's own position included), so older pages can be given back."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request: a tensor of `shape` in `dtype`
    ("float32", or "activation" for the engine's activation dtype), one row per
    request slot.  The mixer resets it when a request's first tokens arrive."""
    shape: tuple
    dtype: str = "float32"
