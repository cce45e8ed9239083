"""Choice and launch of the attention kernels for a step.

bfloat16 steps use the tensor-core prefill kernel for requests that bring more
than one token and the split-key decode kernel for requests that bring exactly
one; both are compiled for the model's head size at first use.  Everything else
(the true 32-bit path) goes to the CUDA-core kernel, which is also the reference
the other two are tested against.
"""
from __future__ import annotations

import functools

from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import ops, scratch
from .build import load_library

DECODE_SPLIT = 256          # keys per split of the decode kernel when nothing chooses (any multiple of 64 will do)
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


_launches: dict = {}        # operands' places and sizes -> (launcher, converted arguments): see prefill_attention


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


SCRATCH = "decode attention partial results"


def _partials(device, floats: int) -> torch.Tensor:
    """Float scratch for the decode kernel's per-split results (see `scratch`)."""
    return scratch.get(device, SCRATCH, floats, at_least=1 << 20)


def reserve_decode(device, max_tokens: int, heads: int, head_dim: int, max_seq_len: int) -> None:
    """Size the scratch for `max_tokens` single-token requests of up to `max_seq_len` keys at the
    shortest split the host ever picks (64 keys)."""
    splits = decode_splits(-(-max_seq_len // 1024) * 1024, 64)
    scratch.reserve(device, SCRATCH, max_tokens * heads * splits * (head_dim + 2))


def decode_splits(max_seq_len: int, split_keys: int = DECODE_SPLIT) -> int:
    return max(1, -(-max_seq_len // split_keys))


def _decode_time(groups: int, length: int, split: int, slots: int, head_dim: int) -> float:
    """Modelled microseconds of the decode kernel and its merge for `groups` (token, key/value
    head) pairs of `length` keys each, cut every `split` keys: the larger of the time to stream
    the keys and values (6.9 TB/s at best, a little less with short splits, and a last split that
    leaves warps of its CTA idle streams that much slower) and the time the CTAs take in rounds
    of `slots` (a CTA by itself: 4 us and 22 ns a key; a last split shorter than the others is
    as long as its busiest warp, a quarter of a split), plus the merge, which reads split after
    split."""
    scale = head_dim / 128.0
    n = -(-length // split)
    last = length - (n - 1) * split
    busy = min(1.0, -(-4 * last // split) / 4.0)            # share of its four warps that a last, shorter split keeps busy
    stream = groups * ((n - 1) * split + last / busy) * 4.0 * head_dim / (6.9e6 * split / (split + 16.0))
    alone = 4.0 + split * 0.022 * scale
    short = 4.0 + min(split, 4 * last) * 0.022 * scale
    whole = groups * (n - 1)                                # CTAs of whole splits, in rounds of `slots`
    rounds = -(-whole // slots)
    left = max(0, groups - (rounds * slots - whole))        # short CTAs that find no place beside them
    in_rounds = rounds * alone + -(-left // slots) * short
    return max(stream, in_rounds) + 0.2 * n


@functools.lru_cache(maxsize=4096)
def decode_split_keys(n_tokens: int, kv_heads: int, max_seq_len: int, num_sms: int = 148,
                      head_dim: int = 128) -> int:
    """Keys per split for a launch, a multiple of 64 up to 1024: the one a small model of the
    kernel's time likes best.  One CTA serves one (token, key/value head, split); three CTAs
    fit an SM, so CTAs run in rounds of 3 x SMs.  Constants fitted to measurements on B200
    (batch 1 to 64, 300 to 4000 keys): the pick is within a few percent of the best there,
    where a fixed 256 keys was 11 % off on average (few CTAs: a round and a bit of small ones
    is worse than one round of larger ones; many: the longer the split the better it streams).

    The answer is the same for all lengths of a stretch of 256 (the model is asked about both
    ends of the stretch), so that a sequence that grows changes its split, and with it the
    rounding of its result and the shape of a captured step, every 256 tokens at most."""
    slots = 3 * num_sms
    groups = n_tokens * kv_heads
    high = -(-max(max_seq_len, 1) // 256) * 256
    low = high - 255
    best_split, best_time = DECODE_SPLIT, None
    for split in range(64, 1025, 64):
        t = _decode_time(groups, low, split, slots, head_dim) + _decode_time(groups, high, split, slots, head_dim)
        if best_time is None or t < best_time:
            best_split, best_time = split, t
    return best_split


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
    # (the same operands in the same places: launched from what the first such call converted; see gemm_tc.gemm)
    key = (q.data_ptr(), q.shape, q.stride(0), q.dtype, out.data_ptr(), out.stride(0), cache_tensor.data_ptr(),
           cache_tensor.shape, cache_tensor.stride(0), block_table.data_ptr(), block_table.stride(0),
           req_start.data_ptr(), req_ctx.data_ptr(), req_qlen.data_ptr(), n_requests, n_tokens, include_single,
           heads, kv_heads, head_dim, window, scale, page_size, variant)
    known = _launches.get(key)
    if known is not None:
        ops._check(known[0](*known[1], ops._stream()), "attention_prefill_tc")
        return
    if variant == 0:
        variant = 2 if tc_prefill_takes(head_dim, page_size) and cache_tensor.is_contiguous() else 1
    if variant == 2:
        from .gemm_tc import status_word

        fn = _prefill_tc_lib(head_dim).fl_attention_prefill_tc
        args = (ops._ptr(q), ops._ld(q), ops._ptr(out), ops._ld(out),
                ops._ptr(cache_tensor), cache_tensor.shape[0], page_size,
                ops._ptr(block_table), block_table.stride(0), ops._ptr(req_start),
                ops._ptr(req_ctx), ops._ptr(req_qlen), n_requests, n_tokens,
                1 if include_single else 0, heads, kv_heads, int(window or 0),
                float(scale), ops._ptr(status_word(q.device)))
        ops._check(fn(*args, ops._stream()), "attention_prefill_tc")
        if len(_launches) > 8192:
            _launches.clear()
        _launches[key] = (fn, args)
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


def num_sms(device) -> int:
    key = ("sms", device)
    if key not in _state:
        _state[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _state[key]


def paged_attention(q, out, cache, step, heads, kv_heads, head_dim, window, scale, split_keys, n_splits):
    """Attention for every token of a bfloat16 step: the decode kernel (its keys cut every
    `split_keys` into `n_splits`) for requests with one token, the prefill kernel for the others."""
    n_dec = step.n_decode_tokens
    if n_dec:
        tok_list = None if n_dec == step.n_tokens else step.decode_tokens
        decode_attention(q, out, cache.tensor, cache.block_table, step.tok_req, step.positions, tok_list,
                         n_dec, heads, kv_heads, head_dim, window, scale, cache.page_size,
                         n_splits, 0, split_keys)
    if n_dec < step.n_tokens:
        prefill_attention(q, out, cache.tensor, cache.block_table, step.req_start, step.req_ctx,
                          step.req_qlen, step.n_requests, step.n_tokens, False, heads, kv_heads,
                          head_dim, window, scale, cache.page_size)
