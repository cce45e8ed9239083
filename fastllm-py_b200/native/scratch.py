"""Scratch memory that kernels of this process share, and the rule that keeps captured
CUDA graphs honest about it.

Two kernels leave results in global memory that is neither an input nor an output of
the step: the split-K products (float partial sums) and the split-key decode attention
(per-split partial results).  Both take a named buffer from here.  A buffer is made
once per device and grows on demand; a captured CUDA graph, however, holds the raw
address of the buffer it was captured with, so a buffer that grew would leave every
older graph writing into memory that has been handed back.  Therefore

  * every growth bumps the device's `generation`; whoever replays graphs stores the
    generation with each graph and drops the graphs of an older one before the next
    replay (`Engine` does);
  * growth during a capture is an error (the step must run once eagerly before);
  * `reserve` lets an engine size the buffers once, up front, from its limits, so
    that in steady use nothing grows at all.

fastllm-py sizes its decode scratch once per captured graph for the same reason
(fastllm_py/graph_decode.py:25-28: every buffer a graph touches is fixed before the
capture).
"""
from __future__ import annotations

import torch

_buffers: dict = {}          # (device, name) -> float32 tensor
_generation: dict = {}       # device -> int


_keys: dict = {}             # any spelling of a device -> its key below (str() of a device is slow)


def _key(device) -> str:
    key = _keys.get(device)
    if key is None:
        key = _keys[device] = str(torch.device(device))
    return key


def generation(device) -> int:
    """Bumped whenever a scratch buffer of `device` was replaced by a larger one."""
    return _generation.get(_key(device), 0)


def bump(device) -> None:
    """Some buffer that captured graphs may point to was replaced."""
    _generation[_key(device)] = generation(device) + 1


def _capturing(device) -> bool:
    return torch.device(device).type == "cuda" and torch.cuda.is_available() \
        and torch.cuda.is_current_stream_capturing()


def get(device, name: str, floats: int, at_least: int = 0) -> torch.Tensor:
    """The float32 buffer `name` of `device` with room for `floats` values."""
    key = (_key(device), name)
    buf = _buffers.get(key)
    if buf is None or buf.numel() < floats:
        if _capturing(device):
            raise RuntimeError(f"scratch buffer {name!r} would have to grow to {floats} floats during "
                               f"graph capture; run the step once eagerly before capturing it")
        replaced = buf is not None
        buf = torch.empty(max(floats, at_least), dtype=torch.float32, device=device)
        _buffers[key] = buf
        if replaced:
            bump(device)
    return buf


def reserve(device, name: str, floats: int) -> None:
    """Make sure `name` holds at least `floats` values (called when an engine is built)."""
    if floats > 0:
        get(device, name, floats)


def size(device, name: str) -> int:
    buf = _buffers.get((_key(device), name))
    return 0 if buf is None else buf.numel()
