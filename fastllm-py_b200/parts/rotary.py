"""Rotary position encoding as a table.

The part turns its constants into cos/sin tables [max_positions, rot_dim/2] in
float32 on the host, once; the attention kernels index them by position.  Any
rotary variant is a different table, so the kernels do not change with it.

Formulas (fastllm_py/kernels/ops.py:77-81, fastllm_py/model.py:329-339):
inv_freq[j] = 1 / theta^(2j / D) in float32; with linear scaling the integer
positions are divided by the factor in float64 and then cast to float32;
angle = position * inv_freq in float32.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part
from .registry import register_part


@register_part("position", "rotary")
class Rotary(Part):
    """params: rot_dim (even, <= head_dim), theta, scaling: None | ("linear", factor)."""
    category = "position"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.rot_dim = int(spec.params["rot_dim"])
        self.theta = float(spec.params["theta"])
        self.scaling = spec.params.get("scaling")
        if self.rot_dim % 2:
            raise ValueError(f"rotary: rot_dim {self.rot_dim} must be even")
        if self.scaling is not None and self.scaling[0] != "linear":
            raise ValueError(f"rotary: scaling {self.scaling[0]!r} is not supported")

    def tables(self):
        """(cos, sin) on the device, shared by all parts with the same constants."""
        key = ("rotary", self.rot_dim, self.theta, self.scaling, self.ctx.max_positions)
        if key not in self.ctx.shared:
            d = self.rot_dim
            inv_freq = 1.0 / (self.theta ** (np.arange(0, d, 2, dtype=np.float32) / d))
            inv_freq = inv_freq.astype(np.float32)
            pos = np.arange(self.ctx.max_positions)
            if self.scaling is not None:
                pos = pos / float(self.scaling[1])
            ang = pos.astype(np.float32)[:, None] * inv_freq[None, :]
            cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(self.ctx.device)
            sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(self.ctx.device)
            self.ctx.shared[key] = (cos.contiguous(), sin.contiguous())
        return self.ctx.shared[key]
