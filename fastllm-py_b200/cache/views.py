"""What a mixer is handed for one run of a step: its layer's share of the cache.

The engine builds these from the cache manager's device tensors and the step's
tables; a mixer never sees the manager itself.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PagedCacheView:
    """For a mixer with a paged need: its layer's pages and this step's tables."""
    tensor: torch.Tensor          # [pages, *need.page_shape(page_size)]
    block_table: torch.Tensor     # [requests in the step, max pages] int32
    slots: torch.Tensor           # [tokens in the step] int32: page * page_size + offset
    page_size: int
    writes: bool                  # False when the run reads another run's cache


@dataclass
class StateView:
    """For a mixer with fixed-size state: one row per request slot."""
    tensor: torch.Tensor          # [request slots, *shape]
    writes: bool
