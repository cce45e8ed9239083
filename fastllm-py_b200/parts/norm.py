"""RMSNorm: x * (mean(x^2) + eps)^-1/2 * w, eps inside the root, the weight
multiplies (no "+1").  fastllm_py/kernels/ops.py:19-27; the fused
residual-add form is fastllm_py/graph_decode.py:300-324."""
from __future__ import annotations

import torch

from ..native import ops
from .base import Part
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: size, eps.  tensors: weight [size]."""
    category = "norm"
    takes_partial = True                 # split-K partial sums are added while the row is read

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def weight_shapes(self):
        return {"weight": (self.size,)}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def apply(self, stream, out, rows=None):
        """Norm the residual stream into `out`, adding the pending sum first.
        With `rows` (int32 indices) only those rows are normed, into out[0..m), and the
        pending sum (a tensor then: `ResidualStream.norm_into` sees to it) stays pending."""
        if stream.pending is not None:
            if not isinstance(stream.pending, torch.Tensor):         # split-K partial sums
                if rows is not None:
                    raise RuntimeError("a gathered norm cannot take partial sums")
                ops.add_rmsnorm_partial(stream.x, stream.pending, self.weight, out, self.eps)
                stream.pending = None
                return
            ops.add_rmsnorm(stream.x, stream.pending, self.weight, out, self.eps, rows)
            if rows is None:
                stream.pending = None
        else:
            ops.rmsnorm(stream.x, self.weight, out, self.eps, rows)
