"""Choice and launch of the attention kernels for a step.

bfloat16 steps use the tensor-core prefill kernel for requests that bring more
than one token and the split-key decode kernel for requests that bring exactly
one; both are compiled for the model's head size at first use.  Everything else
(the true 32-bit path) goes to the CUDA-core kernel, which is also the reference
the other two are tested against.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import ops
from .build import load_library

DECODE_SPLIT = 256          # the smallest split of the decode kernel, in keys (larger ones are multiples)
_libs: dict = {}
_state: dict = {}


def handles(dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


TC_PREFILL_HEAD_DIMS = (64, 128)       # head sizes the tcgen05 prefill kernel is built for


def libraries(head_dim: int) -> list:
    libs = [("attention_decode", {"HEAD_DIM": head_dim}), ("attention_prefill", {"HEAD_DIM": head_dim})]
    if head_dim in TC_PREFILL_HEAD_DIMS:
        libs.append(("attention_prefill_tc", {"HEAD_DIM": head_dim}))
    return libs


def tc_prefill_takes(head_dim: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel's limits: head size 64 or 128, pages of a
    multiple of 8 tokens that divide its 128-key block."""
    return head_dim in TC_PREFILL_HEAD_DIMS and page_size % 8 == 0 and 8 <= page_size <= 128 \
        and 128 % page_size == 0


def _decode_lib(head_dim: int):
    key = ("decode", head_dim)
    lib = _libs.get(key)
    if lib is None:
        lib = load_library("attention_decode", {"HEAD_DIM": head_dim})
        lib.fl_attention_decode.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long,
                                            c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.fl_attention_decode.restype = c_int
        assert lib.fl_attention_decode_head_dim() == head_dim
        assert DECODE_SPLIT % lib.fl_attention_decode_split_unit() == 0
        _libs[key] = lib
    return lib


def _prefill_lib(head_dim: int):
    key = ("prefill", head_dim)
    lib = _libs.get(key)
    if lib is None:
        lib = load_library("attention_prefill", {"HEAD_DIM": head_dim})
        lib.fl_attention_prefill.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long,
                                             c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        lib.fl_attention_prefill.restype = c_int
        assert lib.fl_attention_prefill_head_dim() == head_dim
        _libs[key] = lib
    return lib


def _prefill_tc_lib(head_dim: int):
    key = ("prefill_tc", head_dim)
    lib = _libs.get(key)
    if lib is None:
        lib = load_library("attention_prefill_tc", {"HEAD_DIM": head_dim})
        lib.fl_attention_prefill_tc.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int,
                                                c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
        lib.fl_attention_prefill_tc.restype = c_int
        assert lib.fl_attention_prefill_tc_head_dim() == head_dim
        _libs[key] = lib
    return lib


def _partials(device, floats: int) -> torch.Tensor:
    """Float scratch for the decode kernel's per-split results; grows on demand,
    never inside a graph capture."""
    key = ("partials", str(device))
    ws = _state.get(key)
    if ws is None or ws.numel() < floats:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the decode-attention workspace would have to grow during graph capture")
        ws = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _state[key] = ws
    return ws


def decode_splits(max_seq_len: int, split_keys: int = DECODE_SPLIT) -> int:
    return max(1, -(-max_seq_len // split_keys))


def decode_split_keys(n_tokens: int, kv_heads: int, max_seq_len: int, num_sms: int = 148) -> int:
    """Keys per split for a launch: a CTA streams better the longer its stretch of keys
    (1024-key splits reach 6.5 TB/s where 256-key ones reach 6.0), but only while there are
    CTAs enough for four or five rounds over the GPU (three CTAs fit an SM); with few tokens
    or short sequences the smallest split gives the most CTAs."""
    for split in (1024, 512):
        if n_tokens * kv_heads * -(-max_seq_len // split) >= 14 * num_sms:
            return split
    return DECODE_SPLIT


def decode_attention(q, out, cache_tensor, block_table, tok_req, positions, tok_list, n_list, heads,
                     kv_heads, head_dim, window, scale, page_size, n_splits, variant=0,
                     split_keys=DECODE_SPLIT):
    """Split-key attention for the tokens in tok_list (None: tokens 0..n_list).
    variant 0 chooses (tensor cores when a key/value head serves at most 16 query heads
    and the head size is a multiple of 16), 1 forces the CUDA-core kernel."""
    lib = _decode_lib(head_dim)
    ws = None
    if n_splits > 1:
        ws = _partials(q.device, n_list * heads * n_splits * (head_dim + 2))
    k_ptr = c_void_p(cache_tensor.data_ptr())
    v_ptr = c_void_p(cache_tensor.data_ptr() + cache_tensor.stride(1) * cache_tensor.element_size())
    rc = lib.fl_attention_decode(ops._ptr(q), ops._ld(q), ops._ptr(out), ops._ld(out), k_ptr, v_ptr,
                                 cache_tensor.stride(0), page_size, ops._ptr(block_table),
                                 block_table.stride(0), ops._ptr(tok_req), ops._ptr(positions),
                                 ops._ptr(tok_list), n_list, heads, kv_heads, int(window or 0),
                                 float(scale), n_splits, int(split_keys), ops._ptr(ws), int(variant), ops._stream())
    ops._check(rc, "attention_decode", 2 if n_splits > 1 else 1)


def prefill_attention(q, out, cache_tensor, block_table, req_start, req_ctx, req_qlen, n_requests,
                      n_tokens, include_single, heads, kv_heads, head_dim, window, scale, page_size,
                      variant=0):
    """Tensor-core attention for the requests of the step that bring several tokens.
    variant 0 chooses: the tcgen05 kernel where it applies (2), else mma.sync (1)."""
    if variant == 0:
        variant = 2 if tc_prefill_takes(head_dim, page_size) and cache_tensor.is_contiguous() else 1
    if variant == 2:
        from .gemm_tc import status_word

        lib = _prefill_tc_lib(head_dim)
        rc = lib.fl_attention_prefill_tc(ops._ptr(q), ops._ld(q), ops._ptr(out), ops._ld(out),
                                         ops._ptr(cache_tensor), cache_tensor.shape[0], page_size,
                                         ops._ptr(block_table), block_table.stride(0), ops._ptr(req_start),
                                         ops._ptr(req_ctx), ops._ptr(req_qlen), n_requests, n_tokens,
                                         1 if include_single else 0, heads, kv_heads, int(window or 0),
                                         float(scale), ops._ptr(status_word(q.device)), ops._stream())
        ops._check(rc, "attention_prefill_tc")
        return
    lib = _prefill_lib(head_dim)
    k_ptr = c_void_p(cache_tensor.data_ptr())
    v_ptr = c_void_p(cache_tensor.data_ptr() + cache_tensor.stride(1) * cache_tensor.element_size())
    rc = lib.fl_attention_prefill(ops._ptr(q), ops._ld(q), ops._ptr(out), ops._ld(out), k_ptr, v_ptr,
                                  cache_tensor.stride(0), page_size, ops._ptr(block_table),
                                  block_table.stride(0), ops._ptr(req_start), ops._ptr(req_ctx),
                                  ops._ptr(req_qlen), n_requests, n_tokens, 1 if include_single else 0,
                                  heads, kv_heads, int(window or 0), float(scale), ops._stream())
    ops._check(rc, "attention_prefill")


def paged_attention(q, out, cache, step, heads, kv_heads, head_dim, window, scale):
    """Attention for every token of a bfloat16 step: the decode kernel for
    requests with one token, the prefill kernel for the others."""
    n_dec = step.n_decode_tokens
    if n_dec:
        tok_list = None if n_dec == step.n_tokens else step.decode_tokens
        decode_attention(q, out, cache.tensor, cache.block_table, step.tok_req, step.positions, tok_list,
                         n_dec, heads, kv_heads, head_dim, window, scale, cache.page_size,
                         step.decode_splits, 0, step.decode_split_keys)
    if n_dec < step.n_tokens:
        prefill_attention(q, out, cache.tensor, cache.block_table, step.req_start, step.req_ctx,
                          step.req_qlen, step.n_requests, step.n_tokens, False, heads, kv_heads,
                          head_dim, window, scale, cache.page_size)
