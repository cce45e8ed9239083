"""SwiGLU feed-forward: down( silu(gate(h)) * up(h) ), no biases.

fastllm_py/model.py:432-435 with the activation of
fastllm_py/kernels/ops.py:157-163: g / (1 + exp(-g)) * u in float.  gate and up
are stacked into one matrix so that one product serves both."""
from __future__ import annotations

from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """params: hidden_size, intermediate_size.  tensors: gate, up [I, hidden], down [hidden, I]."""
    category = "feed_forward"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.gate_up = None
        self.down = None

    def weight_shapes(self):
        return {"gate": (self.inter, self.hidden), "up": (self.inter, self.hidden),
                "down": (self.hidden, self.inter)}

    def load(self, tensors):
        if tensors["gate"].dtype != tensors["up"].dtype:
            raise ValueError("swiglu: gate and up matrices must be stored in one dtype")
        self.gate_up = Linear([tensors["gate"], tensors["up"]])
        self.down = Linear([tensors["down"]])

    def reserve(self, limits):
        for lin in (self.gate_up, self.down):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step):
        n = h.shape[0]
        dt = self.ctx.dtype
        act = step.workspace.rows("ffn_act", n, self.inter, dt)
        if self.gate_up.forward_gated(h, act):               # product and activation in one kernel
            return self.down.forward(act, out, defer=True)
        gu = step.workspace.rows("gate_up", n, 2 * self.inter, dt)
        partial = self.gate_up.forward(h, gu, defer=True)
        if partial is None:
            ops.swiglu(gu, act)
        else:
            ops.swiglu_partial(partial, act)
        return self.down.forward(act, out, defer=True)
