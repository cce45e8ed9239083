"""What every part is, and what a part may ask of the engine while it runs.

A part is built from a PartSpec (kind, sizes and constants, tensor names) and a
BuildContext (device, activation dtype, page size).  It declares the shapes of
its tensors by slot, receives them at load, and runs on the tokens of one step.
It knows nothing of the model it is in: names of checkpoint tensors, the number
of layers and the architecture stay in the plan.

Interfaces by category (all tensors are torch CUDA tensors; `step` is the
engine's StepContext; buffers come from `step.workspace`):

  embedding     forward(step, out)            out: [N, hidden] float32 residual stream
  position      tables(max_positions)         -> (cos, sin) float32 [max_positions, rot_dim/2]
  norm          apply(stream, out, rows=None) adds the stream's pending sum, then norms into `out`
  mixer         cache_need() -> PagedKV | FixedState | None
                forward(h, out, step, cache)  h: [N, hidden] -> out: [N, hidden]
  feed_forward  forward(h, out, step)
  block         forward(stream, step, cache)  the arrangement of mixer, feed-forward and norms
  head          forward(h, out)               h: [m, hidden] -> out: [m, vocab] float32
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class BuildContext:
    device: torch.device
    dtype: torch.dtype                 # activation / cache dtype: torch.bfloat16 or torch.float32
    page_size: int
    max_positions: int                 # position tables cover [0, max_positions)
    shared: dict = field(default_factory=dict)   # objects parts may share (position tables by spec)


class Part:
    category = None

    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx

    def weight_shapes(self) -> dict:
        """slot -> expected shape of the checkpoint tensor."""
        return {}

    def load(self, tensors: dict) -> None:
        """Receives slot -> device tensor in its stored dtype."""

    def children(self) -> list:
        """Parts nested inside this one (their tensors are loaded too)."""
        return []


class ResidualStream:
    """The residual sum, float32 in both precisions, plus a sum not yet added.

    A mixer or feed-forward leaves its output as `pending`; the next norm adds
    it while it norms (one pass over the row instead of two), which is the
    deferred add of fastllm_py/graph_decode.py:810-813."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None


class Workspace:
    """Named activation buffers, made once for the most tokens a step may have.

    `rows(name, n, cols, dtype)` returns the first n rows of the buffer of that
    name; parts that run one after another share buffers by using the same
    name.  Row pitch is rounded up to 16 bytes (what a TMA descriptor wants)."""

    def __init__(self, device, max_tokens: int):
        self.device = device
        self.max_tokens = max_tokens
        self._buffers: dict = {}

    def rows(self, name: str, n: int, cols: int, dtype, initial: int | None = None) -> torch.Tensor:
        """`initial` (for buffers that are wide but usually short, like logits)
        starts the buffer at that many rows and lets it grow to max_tokens on demand."""
        key = (name, cols, dtype)
        buf = self._buffers.get(key)
        if n > self.max_tokens:
            raise RuntimeError(f"a step of {n} rows exceeds the workspace's {self.max_tokens}")
        if buf is None or buf.shape[0] < n:
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace buffer {key} would be allocated during graph capture")
            unit = 16 // torch.empty((), dtype=dtype).element_size()
            pitch = -(-cols // unit) * unit
            cap = self.max_tokens if initial is None else min(self.max_tokens, max(initial, n))
            if buf is not None:
                cap = min(self.max_tokens, max(n, 2 * buf.shape[0]))
            buf = torch.zeros((cap, pitch), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:n, :cols]
