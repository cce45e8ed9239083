"""Embedding and output head.

Embedding: x = table[ids], no scaling (fastllm_py/model.py:447).  Head:
logits = x @ W^T in float, no bias, no soft cap (model.py:476); with tied
embeddings the head's matrix is the embedding table itself (model.py:228-231),
which the loader expresses by giving both parts the same tensor."""
from __future__ import annotations

from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("embedding", "table")
class Embedding(Part):
    """params: vocab_size, hidden_size.  tensors: weight [vocab, hidden]."""
    category = "embedding"
    takes_fed_tokens = True              # an id -1 - r is taken from row r of step.token_feed

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.table = None

    def weight_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def load(self, tensors):
        self.table = tensors["weight"]

    def forward(self, step, out):
        ops.embed(self.table, step.token_ids, out, step.status, getattr(step, "token_feed", None))


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab_size, hidden_size.  tensors: weight [vocab, hidden]."""
    category = "head"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.linear = None

    def weight_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def load(self, tensors):
        # a table that the embedding part reads too stays row-major; a matrix of its own may be packed
        w = tensors["weight"]
        self.linear = Linear.sharing(w) if "weight" in self.shared_slots else Linear([w])

    def reserve(self, limits):
        if self.linear is not None:
            self.linear.reserve(self.ctx.dtype, min(limits.max_tokens, limits.max_requests))

    def forward(self, h, out):
        self.linear.forward(h, out)
