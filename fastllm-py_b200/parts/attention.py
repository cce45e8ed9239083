"""Attention mixer: grouped-query causal attention over a paged cache.

Formulas (fastllm_py/model.py:399-430, :341-353): q, k, v = h Wq^T, h Wk^T,
h Wv^T, split head-major; rotary encoding of q and k at the tokens' absolute
positions; the rotated key and the value join the cache; scores
q.k * head_dim^-1/2 over the visible keys (those at or before the query, within
`window` if the layer has one), softmax in float, weighted sum of values, merged
head-major; output projection Wo.  Query head h reads KV head
h // (heads / kv_heads).

One stacked matrix serves q|k|v.  A layer that reads another layer's cache
(`shares_cache`) has no k/v matrices and writes nothing.
"""
from __future__ import annotations

import torch

from ..cache.needs import PagedKV
from ..cache.views import PagedCacheView
from ..native import ops
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("mixer", "attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, position (PartSpec | None),
    window (None | int), shares_cache (bool), scale (None -> head_dim^-1/2).
    tensors: q, o and, unless shares_cache, k, v."""
    category = "mixer"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = p.get("window")
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        if self.heads % self.kv_heads:
            raise ValueError(f"attention: {self.heads} heads are not a multiple of "
                             f"{self.kv_heads} kv heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention: head_dim {self.head_dim} is not supported by the kernels "
                             f"(multiples of 16 from 16 to 256)")
        if self.heads > 65535:
            raise ValueError(f"attention: {self.heads} heads exceed the kernels' limit of 65535")
        self.position = build_part("position", p["position"], ctx) if p.get("position") else None
        self.qkv = None
        self.o = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_need(self):
        if self.shares_cache:
            return None
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    # ---- what the host decides per step: how the decode kernel splits the keys
    @property
    def plan_key(self):
        """Mixers with equal keys take equal decisions, so one of them is asked per step."""
        return ("attention", self.heads, self.kv_heads, self.head_dim)

    def _fast(self):
        from ..native import attention as fast
        return fast if fast.handles(self.ctx.dtype, self.head_dim) else None

    def reserve(self, limits):
        for lin in (self.qkv, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)
        fast = self._fast()
        if fast is not None:
            fast.reserve_decode(self.ctx.device, min(limits.max_tokens, limits.max_requests), self.heads,
                                self.head_dim, limits.max_model_len)

    def plan_step(self, step):
        """(keys per split, splits) of the decode kernel for this step: enough splits for the
        longest sequence.  In a step that may be replayed from a captured graph the splits cover
        the length rounded up to 1024 (CTAs of splits beyond a sequence's end leave at once) and
        the keys per split change every 256 tokens at most, so a graph serves hundreds of steps."""
        fast = self._fast()
        if fast is None or step.n_decode_tokens == 0:
            step.plans[self.plan_key] = (0, 1)             # no launch of that kernel: one answer, one graph key
            return
        longest = step.max_seq_len
        keys = fast.decode_split_keys(step.n_decode_tokens, self.kv_heads, longest, fast.num_sms(self.ctx.device),
                                      self.head_dim)
        if step.for_graph:
            longest = -(-longest // 1024) * 1024
        step.plans[self.plan_key] = (keys, fast.decode_splits(longest, keys))

    def graph_key(self, step):
        return step.plans.get(self.plan_key)

    def weight_shapes(self):
        q_out, kv_out = self.heads * self.head_dim, self.kv_heads * self.head_dim
        shapes = {"q": (q_out, self.hidden), "o": (self.hidden, q_out)}
        if not self.shares_cache:
            shapes["k"] = (kv_out, self.hidden)
            shapes["v"] = (kv_out, self.hidden)
        return shapes

    def load(self, tensors):
        mats = [tensors["q"]] if self.shares_cache else [tensors["q"], tensors["k"], tensors["v"]]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("attention: q, k and v matrices must be stored in one dtype")
        self.qkv = Linear(mats)
        self.o = Linear([tensors["o"]])

    def forward(self, h, out, step, cache: PagedCacheView):
        n = h.shape[0]
        dt = self.ctx.dtype
        q_cols = self.heads * self.head_dim
        cols = q_cols if self.shares_cache else q_cols + 2 * self.kv_heads * self.head_dim
        if cache.writes == self.shares_cache:
            raise RuntimeError("attention: the run's cache and the layer's shares_cache disagree")
        qkv = step.workspace.rows("qkv", n, cols, dt)
        queries = qkv if cols == q_cols else step.workspace.rows("qkv", n, cols, dt, first=q_cols)
        if self.position is not None:
            cos, sin = self.position.tables()
            rot = self.position.rot_dim
        else:
            cos, sin, rot = step.no_rotation, step.no_rotation, 0
        kv_cache = cache.tensor if cache.writes else None
        # prompt-sized steps of a layer with heads of 128: product, rotation and cache write in one kernel
        fused = kv_cache is not None and rot == self.head_dim and self.qkv.forward_qkv_rope(
            h, queries, self.heads, self.kv_heads, self.head_dim, rot, cos, sin, step.positions,
            cache.slots, kv_cache, cache.page_size)
        if not fused:
            partial = self.qkv.forward(h, qkv, defer=True)
            if partial is None:
                ops.rope_kv_write(qkv, self.heads, self.kv_heads, self.head_dim, rot, cos, sin,
                                  step.positions, cache.slots, kv_cache, cache.page_size)
            else:
                ops.rope_kv_write_partial(partial, queries, self.heads, self.kv_heads, self.head_dim,
                                          rot, cos, sin, step.positions, cache.slots, kv_cache,
                                          cache.page_size)
        ctx = step.workspace.rows("attn_ctx", n, q_cols, dt)
        self.attend(queries, ctx, step, cache)
        return self.o.forward(ctx, out, defer=True)

    def attend(self, q, ctx, step, cache):
        fast = self._fast()
        if fast is not None:
            if self.plan_key not in step.plans:           # a step built by hand, not by the engine
                self.plan_step(step)
            keys, splits = step.plans[self.plan_key]
            fast.paged_attention(q, ctx, cache, step, self.heads, self.kv_heads, self.head_dim,
                                 self.window, self.scale, keys, splits)
        else:
            ops.paged_attention_simt(q, ctx, cache.tensor, cache.block_table, step.tok_req,
                                     step.positions, self.heads, self.kv_heads, self.head_dim,
                                     self.window, self.scale, cache.page_size)
