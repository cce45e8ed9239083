"""What a mixer asks of the cache manager.

A mixer declares its need; the manager groups equal needs and serves each group
from pages of its own.  fastllm-py has one kind only (every layer keeps all keys
and values, fastllm_py/model.py:76-123), so it has no such notion.

A paged need says what one page looks like and what a token costs; the manager
hands out pages and block tables and never looks inside a page.  Another paged
layout (one latent vector per token, say) is another subclass of `PagedNeed`;
nothing in the manager changes for it.
"""
from __future__ import annotations

from dataclasses import dataclass


class PagedNeed:
    """Per-token storage in pages.  Subclasses are frozen dataclasses (equal needs share a
    group of pages) with an attribute `window` (None: every token is kept; a number: the
    last `window` tokens, the query's own position included, so older pages can go back) and

        page_shape(page_size) -> tuple   shape of one page of one layer, in elements
        dtype                            "activation" (the engine's activation dtype) or a torch dtype name
    """
    window = None
    dtype = "activation"

    def page_shape(self, page_size: int) -> tuple:
        raise NotImplementedError

    def bytes_per_token(self, page_size: int, itemsize: int) -> int:
        """Cache bytes one token costs in one layer with this need (`itemsize`: of the
        engine's activation dtype, used when the need stores activations)."""
        if self.dtype != "activation":
            import torch

            itemsize = torch.empty((), dtype=getattr(torch, self.dtype)).element_size()
        elements = 1
        for d in self.page_shape(page_size):
            elements *= int(d)
        return elements * itemsize // page_size


@dataclass(frozen=True)
class PagedKV(PagedNeed):
    """Keys and values per token: `kv_heads` x `head_dim` each, a page laid out as
    [2 (keys, values), kv_heads, page_size, head_dim], so that the page_size x head_dim
    tile of one head of one page is contiguous."""
    kv_heads: int
    head_dim: int
    window: int | None = None

    def page_shape(self, page_size: int) -> tuple:
        return (2, self.kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request: a tensor of `shape` in `dtype`
    ("float32", or "activation" for the engine's activation dtype), one row per
    request slot.  The mixer resets it when a request's first tokens arrive."""
    shape: tuple
    dtype: str = "float32"
