"""Linear: out = a @ W^T for an (out_features, in_features) weight, no bias.

fastllm-py keeps every projection as its own (out, in) array and calls cuBLAS
(`matmul_w`, fastllm_py/model.py:55-63).  Here a Linear may hold several
checkpoint matrices stacked along the output axis (q|k|v, gate|up), so that one
product serves them all, and picks the kernel by operand types:

  * bfloat16 activations and bfloat16 weights: the tcgen05 tensor-core kernels.
    At its first such product the Linear packs its matrix by k-block, the layout
    those kernels stream fastest (native/gemm_tc.py: PackedWeight), and lets the
    row-major copy go, unless something else reads that copy too (a tied
    embedding table);
  * anything with a 32-bit operand: the CUDA-core kernel with float
    accumulation (a weight stored in 32-bit stays 32-bit; the true 32-bit path
    never touches a reduced-precision matrix mode).
"""
from __future__ import annotations

import torch

from ..native import ops


_gemm_tc_module = None


def _gemm_tc():
    """native/gemm_tc.py, imported when a bfloat16 product first needs it (it compiles its library)."""
    global _gemm_tc_module
    if _gemm_tc_module is None:
        from ..native import gemm_tc
        _gemm_tc_module = gemm_tc
    return _gemm_tc_module


class Linear:
    def __init__(self, weights: list):
        """`weights`: matrices [out_i, in] of one dtype, stacked along out."""
        w = weights[0] if len(weights) == 1 else torch.cat(weights, dim=0)
        self.weight = w.contiguous()          # row-major; None once the tensor-core copy has replaced it
        self._set_shape(self.weight)
        self.shared = False
        self._tc = None

    @classmethod
    def sharing(cls, weight: torch.Tensor) -> "Linear":
        """A Linear over an existing tensor without copying it (tied embeddings)."""
        self = cls.__new__(cls)
        self.weight = weight
        self._set_shape(weight)
        self.shared = True
        self._tc = None
        return self

    def _set_shape(self, w: torch.Tensor) -> None:
        self.out_features, self.in_features = w.shape
        self.dtype, self.device = w.dtype, w.device

    def forward(self, a: torch.Tensor, out: torch.Tensor, defer: bool = False):
        """Writes `out` and returns None; or, with `defer`, may leave the product
        as split-K partial sums and return them (a `gemm_tc.Partial`) for a
        consumer that adds them as it reads: `out` is then not written."""
        if a.dtype == torch.bfloat16 and self.dtype == torch.bfloat16:
            return self._tensor_core().forward(a, out, defer)
        if self.weight is None:
            raise ops.KernelError("this Linear's matrix was packed for bfloat16 activations; it cannot "
                                  "serve 32-bit activations as well")
        ops.gemm_simt(a, self.weight, out)
        return None

    def _tensor_core(self):
        if self._tc is None:
            from ..native.gemm_tc import TensorCoreLinear
            self._tc = TensorCoreLinear(self.weight, pack=not self.shared)
            if not self.shared:
                self.weight = None             # the packed copy is the matrix from here on
        return self._tc

    def reserve(self, activation_dtype, max_tokens: int) -> None:
        """Called when an engine is built: make the matrix ready for the kernels that will read it
        (pack it, for bfloat16 products) and size the scratch memory that products of up to
        `max_tokens` rows will take, so that nothing has to grow (and no captured graph goes
        stale) once the engine runs."""
        if activation_dtype == torch.bfloat16 and self.dtype == torch.bfloat16:
            from ..native import gemm_tc
            self._tensor_core()
            gemm_tc.reserve(self.device, self.out_features, self.in_features, max_tokens)

    def forward_qkv_rope(self, a: torch.Tensor, q_out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         rot_dim: int, cos, sin, positions, slots, cache, page_size: int) -> bool:
        """For a Linear that stacks q, k and v matrices: the product with the rotary encoding and the
        cache write in its epilogue (rotated queries into `q_out`, rotated keys and values into the
        tokens' cache slots), in one tensor-core kernel.  False (nothing done) when that kernel does
        not apply; the caller then takes `forward` and the rotary kernel."""
        if a.dtype == torch.bfloat16 and self.dtype == torch.bfloat16:
            return _gemm_tc().gemm_qkv_rope(a, self._tensor_core().weight, q_out, n_heads, n_kv_heads, head_dim, rot_dim,
                                 cos, sin, positions, slots, cache, page_size)
        return False

    def forward_gated(self, a: torch.Tensor, out: torch.Tensor) -> bool:
        """For a Linear that stacks a gate and an up matrix: out = silu(a gate^T) * (a up^T)
        in one tensor-core kernel.  False (nothing done) when that kernel does not apply; the
        caller then takes `forward` and the activation kernel."""
        if a.dtype == torch.bfloat16 and self.dtype == torch.bfloat16:
            return _gemm_tc().gemm_swiglu(a, self._tensor_core().weight, out)
        return False
