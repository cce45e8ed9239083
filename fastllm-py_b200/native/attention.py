"""Choice of the attention kernel for a step.

The CUDA-core kernel (csrc/attention_simt.cu) serves the true 32-bit path and
is the reference for the others.  bfloat16 steps go to the tensor-core prefill
kernel and the split-key decode kernel once those are built for the head size.
"""
from __future__ import annotations

import torch


def handles(dtype, head_dim: int) -> bool:
    return False


def paged_attention(q, out, cache, step, heads, kv_heads, head_dim, window, scale):
    raise NotImplementedError
