"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

"prenorm" is the Llama layer (fastllm_py/model.py:464-470):
    x = x + mixer(norm_mixer(x));  x = x + feed_forward(norm_ff(x))
The sums are left pending on the residual stream and folded into the next norm.
"""
from __future__ import annotations

from .base import Part
from .registry import build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    """norm roles: "mixer", "feed_forward"."""
    category = "block"

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer = build_part("mixer", layer_spec.mixer, ctx)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, ctx)
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], ctx)
        self.norm_ff = build_part("norm", layer_spec.norms["feed_forward"], ctx)
        self.hidden = self.norm_mixer.size

    def children(self):
        return [self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff]

    def forward(self, stream, step, cache):
        n = stream.x.shape[0]
        dt = self.ctx.dtype
        h = step.workspace.rows("normed", n, self.hidden, dt)
        delta = step.workspace.rows("delta", n, self.hidden, dt)
        # a mixer or feed-forward returns None when it wrote `delta`, or the
        # split-K partial sums of its last product, which the next norm adds up
        stream.norm_into(self.norm_mixer, h)
        left = self.mixer.forward(h, delta, step, cache)
        stream.pending = delta if left is None else left
        stream.norm_into(self.norm_ff, h)
        left = self.feed_forward.forward(h, delta, step)
        stream.pending = delta if left is None else left
