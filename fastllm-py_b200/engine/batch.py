"""StepContext: one step's batch as the parts see it, and the buffers behind it.

A step is a flat list of N tokens from n requests; request r brings q_len[r]
consecutive new tokens (a whole prompt, a portion of one, or one decoded token)
at positions ctx_len[r] .. ctx_len[r] + q_len[r] - 1.  fastllm-py has three
separate entry points for one sequence of any length, one token of one
sequence, and one token of each of B slots (fastllm_py/model.py:437,
fastllm_py/graph_decode.py:987, fastllm_py/batched.py:220); this one batch form
covers all of them and their mixtures.

All integer inputs of a step live in ONE pinned host array mirrored by ONE
device array at fixed offsets, so a step costs one host-to-device copy for the
per-token part and one for the block tables, and the device addresses never
change (which is what a captured CUDA graph needs: fastllm-py learned that
inputs must be written on the capture stream into fixed buffers,
fastllm_py/graph_decode.py:25-28).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.views import PagedCacheView, StateView


class StepBuffers:
    """Fixed host/device integer buffers for the largest step the engine allows."""

    def __init__(self, device, max_tokens: int, max_requests: int, n_groups: int, bt_stride: int):
        self.max_tokens, self.max_requests = max_tokens, max_requests
        self.n_groups, self.bt_stride = n_groups, bt_stride
        T, R = max_tokens, max_requests
        layout = [("token_ids", T), ("positions", T), ("tok_req", T), ("logit_rows", T),
                  ("decode_tokens", T)]
        layout += [(f"slots{g}", T) for g in range(n_groups)]
        layout += [("req_start", R + 1), ("req_ctx", R), ("req_qlen", R), ("req_slot", R)]
        self.offsets = {}
        off = 0
        for name, size in layout:
            self.offsets[name] = (off, size)
            off += -(-size // 4) * 4                      # keep every section 16-byte aligned
        self.small_size = off
        for g in range(n_groups):
            self.offsets[f"bt{g}"] = (off, R * bt_stride)
            off += -(-(R * bt_stride) // 4) * 4
        self.total = off
        pin = torch.cuda.is_available()
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self.copied = None                                # event after the last upload
        self.uploaded_bytes = 0                           # host-to-device bytes copied so far

    def host_view(self, name):
        off, size = self.offsets[name]
        return self.host_np[off:off + size]

    def dev_view(self, name):
        off, size = self.offsets[name]
        return self.dev[off:off + size]

    def wait_for_last_upload(self):
        if self.copied is not None:
            self.copied.synchronize()

    def upload(self, n_requests: int):
        """Per-token section whole; block tables for the first `n_requests` rows
        (0 when no row changed since the last upload)."""
        self.dev[:self.small_size].copy_(self.host[:self.small_size], non_blocking=True)
        self.uploaded_bytes += 4 * self.small_size
        for g in range(self.n_groups):
            if n_requests == 0:
                break
            off, _ = self.offsets[f"bt{g}"]
            used = n_requests * self.bt_stride
            self.dev[off:off + used].copy_(self.host[off:off + used], non_blocking=True)
            self.uploaded_bytes += 4 * used
        if self.dev.is_cuda:
            self.copied = torch.cuda.Event()
            self.copied.record()


@dataclass
class StepContext:
    """The view of one step that parts receive."""
    n_tokens: int
    n_requests: int
    n_wanted: int
    token_ids: torch.Tensor        # [N] int32
    positions: torch.Tensor        # [N] int32 absolute position of each token
    tok_req: torch.Tensor          # [N] int32 index of the token's request in this step
    logit_rows: torch.Tensor       # [m] int32 rows whose logits are wanted
    req_start: torch.Tensor        # [n+1] int32 first row of each request
    req_ctx: torch.Tensor          # [n] int32 tokens already cached before the step
    req_qlen: torch.Tensor         # [n] int32 tokens of the request in this step
    req_slot: torch.Tensor         # [n] int32 state slot of each request
    decode_tokens: torch.Tensor    # [n_decode_tokens] int32 rows of requests that bring exactly one token
    status: torch.Tensor           # [1] int32 device-side error word (0 = fine)
    workspace: object
    no_rotation: torch.Tensor      # stand-in table for mixers without position encoding
    # host copies, for choosing kernels and launch shapes
    q_lens: list = field(default_factory=list)
    ctx_lens: list = field(default_factory=list)
    slots_host: list = field(default_factory=list)
    max_q_len: int = 0
    max_seq_len: int = 0
    rows_identity: bool = False    # the wanted rows are all rows, in order
    n_decode_tokens: int = 0       # tokens of requests that bring exactly one token
    for_graph: bool = False        # the step may be captured or replayed as a CUDA graph
    plans: dict = field(default_factory=dict)   # what mixers decided on the host for this step (plan_step)
    token_feed: object = None      # int32 device tensor: a token id -1 - r stands for token_feed[r]
    _views: dict = field(default_factory=dict)

    def cache_view(self, cache_id: int, writes: bool):
        view = self._views.get(cache_id)
        if view is None:
            return None
        if view.writes != writes:
            view = type(view)(**{**view.__dict__, "writes": writes})
        return view


def build_views(cache, buffers: StepBuffers, n_tokens: int, n_requests: int) -> dict:
    """cache id -> view for this step, over the engine's fixed device buffers."""
    views = {}
    for gi, group in enumerate(cache.groups):
        bt = buffers.dev_view(f"bt{gi}").view(buffers.max_requests, buffers.bt_stride)
        slots = buffers.dev_view(f"slots{gi}")[:n_tokens]
        for cid in group.cache_ids:
            views[cid] = PagedCacheView(group.tensors[cid], bt, slots, cache.page_size, True)
    for cid, tensor in cache.state_tensors.items():
        views[cid] = StateView(tensor, True)
    return views
