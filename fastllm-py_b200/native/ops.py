"""Python faces of the CUDA launchers: torch tensors in, one kernel launch each.

Every function launches on torch's current stream, allocates nothing (outputs
are passed in) and raises if the launch fails.  There is no other
implementation behind these names: without the compiled libraries they raise.
Tensors must live on the CUDA device; strides are passed as leading dimensions,
so row-padded buffers and column slices of wider buffers are fine as long as
the last dimension is contiguous.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream():
    """The current CUDA stream's handle for a launch.  `torch.cuda.current_stream()` asks the
    driver how many devices there are on every call (20 us): a step launched kernel by kernel
    spent more time there than on its kernels, so the raw handle is asked for instead."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _ld(t: torch.Tensor) -> int:
    """Leading dimension (elements between rows) of a 2-D view with a dense last axis."""
    if t.dim() != 2:
        raise KernelError(f"expected a 2-D tensor, got shape {tuple(t.shape)}")
    if t.shape[1] > 1 and t.stride(1) != 1:
        raise KernelError("the last dimension must be contiguous")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


class _Counter:
    """Kernels launched by this process through these wrappers (a graph replay
    adds the number of kernels captured in it)."""
    launches = 0


counter = _Counter()


def _check(rc: int, what: str, kernels: int = 1) -> None:
    if rc != 0:
        raise KernelError(f"{what}: CUDA error {rc} at launch")
    counter.launches += kernels


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")


_fns: dict = {}
_launches: dict = {}        # operands' places and sizes -> (launcher, converted arguments) of wrappers that remember


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    """The launcher `fn_name` of a library with its signature set, looked up once (a step calls
    these wrappers a few hundred times and is short of host time when its kernels are small)."""
    if defines is None:
        fn = _fns.get(fn_name)
        if fn is not None:
            return fn
    key = (lib_name, tuple(sorted((defines or {}).items())), fn_name)
    fn = _fns.get(key)
    if fn is None:
        fn = getattr(load_library(lib_name, defines), fn_name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fns[key] = fn
        if defines is None:
            _fns[fn_name] = fn
    return fn


# ---------------------------------------------------------------- elementwise

def embed(table, ids, out, status, fed=None):
    """out[t] = table[ids[t]] as float32; an id outside the table sets status[0] = t + 1.
    With `fed` (int32 on the device), an id -1 - r is replaced by fed[r]."""
    _require_cuda(table, ids, out, status, fed)
    fn = _fn("elementwise", "fl_embed", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_long, c_int,
                                         c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    if out.dtype != torch.float32 or ids.dtype != torch.int32 or (fed is not None and fed.dtype != torch.int32):
        raise KernelError("embed: out must be float32, ids (and fed) int32")
    _check(fn(_ptr(table), dtype_code(table), _ld(table), _ptr(ids), _ptr(out), _ld(out),
              ids.numel(), table.shape[1], table.shape[0], _ptr(status), _ptr(fed),
              0 if fed is None else fed.numel(), _stream()), "embed")


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight."""
    _require_cuda(x, weight, out, rows)
    fn = _fn("elementwise", "fl_rmsnorm", [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int,
                                           c_long, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(x), dtype_code(x), _ld(x), _ptr(weight), dtype_code(weight), _ptr(out),
              dtype_code(out), _ld(out), out.shape[0], x.shape[1], float(eps), _ptr(rows), _stream()),
           "rmsnorm")


def add_rmsnorm(resid, delta, weight, out, eps, rows=None):
    """resid += delta (float32, written back unless rows are gathered); out = rmsnorm(resid) * weight."""
    _require_cuda(resid, delta, weight, out, rows)
    if resid.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    fn = _fn("elementwise", "fl_add_rmsnorm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p,
                                               c_int, c_void_p, c_int, c_long, c_int, c_int, c_float,
                                               c_void_p, c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(delta), dtype_code(delta), _ld(delta), _ptr(weight),
              dtype_code(weight), _ptr(out), dtype_code(out), _ld(out), out.shape[0], resid.shape[1],
              float(eps), _ptr(rows), _stream()), "add_rmsnorm")


def add_rmsnorm_partial(resid, partial, weight, out, eps):
    """resid += (split-K partial sums, added in slab order); out = rmsnorm(resid) * weight."""
    partial.check()
    # (the same operands in the same places, as in every layer of every step of a size: launched from
    # what the first such call converted; see gemm_tc.gemm)
    key = ("add_rmsnorm_partial", resid.data_ptr(), resid.shape, resid.stride(0), partial.data.data_ptr(),
           partial.splits, partial.split_stride, partial.ld, weight.data_ptr(), weight.dtype, out.data_ptr(),
           out.shape, out.stride(0), out.dtype, eps)
    known = _launches.get(key)
    if known is not None:
        _check(known[0](*known[1], _stream()), "add_rmsnorm_partial")
        return
    _require_cuda(resid, weight, out)
    fn = _fn("elementwise", "fl_add_rmsnorm_partial", [c_void_p, c_long, c_void_p, c_int, c_long, c_long,
                                                       c_void_p, c_int, c_void_p, c_int, c_long, c_int,
                                                       c_int, c_float, c_void_p])
    args = (_ptr(resid), _ld(resid), _ptr(partial.data), partial.splits, partial.split_stride,
            partial.ld, _ptr(weight), dtype_code(weight), _ptr(out), dtype_code(out), _ld(out),
            out.shape[0], resid.shape[1], float(eps))
    _check(fn(*args, _stream()), "add_rmsnorm_partial")
    if len(_launches) > 8192:
        _launches.clear()
    _launches[key] = (fn, args)


def swiglu_partial(partial, out):
    """swiglu over gate|up columns given as split-K partial sums."""
    _require_cuda(out)
    partial.check()
    fn = _fn("elementwise", "fl_swiglu_partial", [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_long,
                                                  c_int, c_int, c_void_p])
    _check(fn(_ptr(partial.data), partial.splits, partial.split_stride, partial.ld, _ptr(out),
              dtype_code(out), _ld(out), out.shape[0], out.shape[1], _stream()), "swiglu_partial")


def rope_kv_write_partial(partial, q_out, n_heads, n_kv_heads, head_dim, rot_dim, cos, sin, positions,
                          slots, cache, page_size):
    """rope_kv_write reading q|k|v as split-K partial sums; rotated queries go to q_out."""
    _require_cuda(q_out, cos, sin, positions, slots, cache)
    partial.check()
    fn = _fn("rope_kv", "fl_rope_kv_write_partial",
             [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p])
    if cache is not None:
        if cache.dtype != q_out.dtype:
            raise KernelError("rope_kv_write: cache and activations must have one dtype")
        k_ptr = c_void_p(cache.data_ptr())
        v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
        page_stride = cache.stride(0)
    else:
        k_ptr = v_ptr = None
        page_stride = 0
    _check(fn(_ptr(partial.data), partial.splits, partial.split_stride, partial.ld, _ptr(q_out),
              dtype_code(q_out), _ld(q_out), q_out.shape[0], n_heads, n_kv_heads, head_dim, rot_dim,
              _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), k_ptr, v_ptr, page_stride, page_size,
              0 if cache is None else 1, _stream()), "rope_kv_write_partial")


def residual_add(resid, delta):
    _require_cuda(resid, delta)
    if resid.dtype != torch.float32:
        raise KernelError("residual_add: the residual stream must be float32")
    fn = _fn("elementwise", "fl_residual_add", [c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int,
                                                c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(delta), dtype_code(delta), _ld(delta), resid.shape[0],
              resid.shape[1], _stream()), "residual_add")


def swiglu(gate_up, out):
    """out[:, i] = silu(gate_up[:, i]) * gate_up[:, I + i], I = out.shape[1]."""
    _require_cuda(gate_up, out)
    if gate_up.dtype != out.dtype:
        raise KernelError("swiglu: input and output must have one dtype")
    fn = _fn("elementwise", "fl_swiglu", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int,
                                          c_void_p])
    _check(fn(_ptr(gate_up), dtype_code(gate_up), _ld(gate_up), _ptr(out), _ld(out), out.shape[0],
              out.shape[1], _stream()), "swiglu")


# -------------------------------------------------------------- rope + cache

def rope_kv_write(qkv, n_heads, n_kv_heads, head_dim, rot_dim, cos, sin, positions, slots, cache,
                  page_size):
    """Rotate q in place; rotate k and copy v of each token into its cache slot.

    `cache` is one layer's [pages, 2, kv_heads, page_size, head_dim] tensor, or
    None when the rows hold queries only (a layer that reads another's cache)."""
    _require_cuda(qkv, cos, sin, positions, slots, cache)
    fn = _fn("rope_kv", "fl_rope_kv_write", [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_long, c_int, c_int, c_void_p])
    if cache is not None:
        if cache.dtype != qkv.dtype:
            raise KernelError("rope_kv_write: cache and activations must have one dtype")
        k_ptr = c_void_p(cache.data_ptr())
        v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
        page_stride = cache.stride(0)
    else:
        k_ptr = v_ptr = None
        page_stride = 0
    _check(fn(_ptr(qkv), dtype_code(qkv), _ld(qkv), qkv.shape[0], n_heads, n_kv_heads, head_dim,
              rot_dim, _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), k_ptr, v_ptr, page_stride,
              page_size, 0 if cache is None else 1, _stream()), "rope_kv_write")


# ------------------------------------------------------------------ attention

def paged_attention_simt(q, out, cache, block_table, tok_req, positions, n_heads, n_kv_heads,
                         head_dim, window, scale, page_size):
    """Causal attention of every token in q over its request's cached keys (CUDA cores)."""
    _require_cuda(q, out, cache, block_table, tok_req, positions)
    if head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} is beyond the kernel's limit of 256")
    fn = _fn("attention_simt", "fl_paged_attention_simt",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long, c_int, c_void_p,
              c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    k_ptr = c_void_p(cache.data_ptr())
    v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), k_ptr, v_ptr, cache.stride(0),
              page_size, _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions),
              q.shape[0], n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _stream()),
           "paged_attention_simt")


# ----------------------------------------------------------------------- GEMM

def gemm_simt(a, w, out):
    """out[M, N] = a[M, K] @ w[N, K]^T, float accumulation on CUDA cores, any dtypes."""
    _require_cuda(a, w, out)
    if a.shape[1] != w.shape[1] or out.shape[0] != a.shape[0] or out.shape[1] != w.shape[0]:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_simt", "fl_gemm_simt", [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_void_p,
                                           c_int, c_long, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), dtype_code(a), _ld(a), _ptr(w), dtype_code(w), _ld(w), _ptr(out),
              dtype_code(out), _ld(out), a.shape[0], w.shape[0], a.shape[1], _stream()), "gemm_simt")


# ------------------------------------------------------------------- sampling

def sample(logits, out, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None):
    """One token per logits row into `out` (int32); null temperature = greedy everywhere."""
    _require_cuda(logits, out, temperature, top_k, top_p, min_p, uniform)
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample: logits must be float32 and out int32")
    if temperature is not None and uniform is None:
        raise KernelError("sample: temperature sampling needs uniform numbers")
    fn = _fn("sampling", "fl_sample", [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), logits.shape[0], logits.shape[1], _ptr(temperature),
              _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out), _stream()), "sample")


def apply_penalties(logits, rows, tokens, counts, repetition, frequency, presence):
    _require_cuda(logits, rows, tokens, counts, repetition, frequency, presence)
    fn = _fn("sampling", "fl_apply_penalties", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                                c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), _ptr(rows), _ptr(tokens), _ptr(counts), rows.numel(),
              _ptr(repetition), _ptr(frequency), _ptr(presence), logits.shape[1], _stream()),
           "apply_penalties")


# ---------------------------------------------------------------------- build

BASE_LIBRARIES = ["elementwise", "rope_kv", "attention_simt", "gemm_simt", "sampling"]
BF16_LIBRARIES = ["gemm_tcgen05"]
