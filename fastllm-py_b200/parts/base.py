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
  mixer         cache_need() -> a need of cache.needs (paged, fixed state) | None
                forward(h, out, step, cache)  h: [N, hidden] -> out: [N, hidden]
  feed_forward  forward(h, out, step)
  block         forward(stream, step, cache)  the arrangement of mixer, feed-forward and norms
  head          forward(h, out)               h: [m, hidden] -> out: [m, vocab] float32

What a part may declare beside its interface (all optional; absent means "no"):

  reserve(limits)          any part: called once when an engine is built, with the most tokens
                           of a step, the most live requests and the longest sequence, so that
                           the part can size the scratch memory its kernels take
  plan_step(step)          mixer: called once per step before anything is launched; decides on
                           the host what the step's launches need (a split of the keys, say) and
                           keeps it in `step.plans`; mixers with an equal `plan_key` are asked once
  graph_key(step)          mixer: what of that plan fixes the launch shapes (part of the key
                           under which a captured step is replayed)
  graph_safe = False       any part whose forward decides on the host from the step's host copies
  takes_partial = True     norm: `apply` accepts split-K partial sums as the stream's pending sum
                           (otherwise the stream adds them up into a tensor first)
  takes_fed_tokens = True  embedding: understands a token id -1 - r as "row r of `step.token_feed`"
                           (without it the scheduler never launches a step ahead of the host)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class EngineLimits:
    """The bounds an engine was built with, as parts see them in `reserve`."""
    max_tokens: int          # tokens of one step
    max_requests: int        # live requests (and so requests of one step)
    max_model_len: int       # longest sequence


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

    shared_slots: frozenset = frozenset()    # set by the decoder before `load`: slots whose tensor another part holds too

    def load(self, tensors: dict) -> None:
        """Receives slot -> device tensor in its stored dtype.  A tensor of a slot in
        `shared_slots` belongs to another part as well and must be left as it is."""

    def children(self) -> list:
        """Parts nested inside this one (their tensors are loaded too)."""
        return []

    def reserve(self, limits: EngineLimits) -> None:
        """Size whatever scratch memory this part's kernels take for steps within `limits`."""


class ResidualStream:
    """The residual sum, float32 in both precisions, plus a sum not yet added.

    A mixer or feed-forward leaves its output as `pending`; the next norm adds
    it while it norms (one pass over the row instead of two), which is the
    deferred add of fastllm_py/graph_decode.py:810-813.  The pending sum is a
    tensor [N, hidden], or the split-K partial sums of the product that made it
    (an object with `reduce_into(tensor)`): a norm that says `takes_partial`
    adds the slabs while it reads, any other gets them added up first, into the
    buffer that `spill()` returns."""

    def __init__(self, x: torch.Tensor, spill=None):
        self.x = x
        self.pending = None
        self.spill = spill

    def norm_into(self, norm, out, rows=None):
        """`norm.apply(self, out, rows)`, with a pending sum that the norm can take."""
        pending = self.pending
        if pending is not None and not isinstance(pending, torch.Tensor):
            if rows is not None or not getattr(norm, "takes_partial", False):
                self.pending = pending.reduce_into(self.spill())
        norm.apply(self, out, rows)


class Workspace:
    """Named activation buffers, made once for the most tokens a step may have.

    `rows(name, n, cols, dtype)` returns the first n rows of the buffer of that
    name; parts that run one after another share buffers by using the same
    name.  Row pitch is rounded up to 16 bytes (what a TMA descriptor wants)."""

    def __init__(self, device, max_tokens: int):
        self.device = device
        self.max_tokens = max_tokens
        self._buffers: dict = {}
        self._views: dict = {}           # (name, cols, dtype, n) -> the view handed out for it before
        self.generation = 0              # bumped when a buffer is replaced by a larger one

    def rows(self, name: str, n: int, cols: int, dtype, initial: int | None = None,
             first: int | None = None) -> torch.Tensor:
        """`initial` (for buffers that are wide but usually short, like logits)
        starts the buffer at that many rows and lets it grow to max_tokens on demand.
        `first`: only the first so many of the `cols` columns (the same memory as the
        whole rows: the queries of a q|k|v buffer, say)."""
        if first is not None:
            view = self._views.get((name, cols, dtype, n, first))
            if view is None:
                whole = self.rows(name, n, cols, dtype, initial)
                view = self._views[(name, cols, dtype, n, first)] = whole[:, :first]
            return view
        view = self._views.get((name, cols, dtype, n))
        if view is not None:             # (making a view costs a few microseconds: a step asks a hundred times)
            return view
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
                self.generation += 1     # captured graphs may hold the old buffer's address
            buf = torch.zeros((cap, pitch), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            for k in [k for k in self._views if k[:3] == key]:
                del self._views[k]
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[(name, cols, dtype, n)] = buf[:n, :cols]
        return view
