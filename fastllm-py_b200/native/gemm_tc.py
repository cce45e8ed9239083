"""The tcgen05 tensor-core product behind `Linear` for bfloat16 operands."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_void_p

import torch

from . import ops, scratch
from .build import load_library

_state: dict = {}


def _lib():
    lib = _state.get("lib")
    if lib is None:
        lib = load_library("gemm_tcgen05")
        lib.fl_gemm_tc.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_long, c_int,
                                   c_int, c_int, c_int, c_int, c_void_p, c_long, c_int, c_void_p,
                                   c_void_p]
        lib.fl_gemm_tc.restype = c_int
        lib.fl_gemm_tc_partial.argtypes = lib.fl_gemm_tc.argtypes
        lib.fl_gemm_tc_partial.restype = c_int
        lib.fl_gemm_tc_plan.argtypes = [c_int, c_int, c_int, c_int, ctypes.POINTER(c_int),
                                        ctypes.POINTER(c_int)]
        lib.fl_gemm_tc_plan.restype = None
        lib.fl_gemm_tc_plan_for.argtypes = [c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int),
                                            ctypes.POINTER(c_int)]
        lib.fl_gemm_tc_plan_for.restype = None
        lib.fl_gemm_tc_swiglu.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                          c_int, c_int, c_void_p, c_void_p]
        lib.fl_gemm_tc_swiglu.restype = c_int
        lib.fl_gemm_tc_qkv_rope.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_long, c_int, c_int, c_void_p, c_void_p]
        lib.fl_gemm_tc_qkv_rope.restype = c_int
        lib.fl_pack_weight.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p]
        lib.fl_pack_weight.restype = c_int
        lib.fl_splitk_reduce.argtypes = [c_void_p, c_long, c_int, c_void_p, c_int, c_long, c_int, c_int, c_void_p]
        lib.fl_splitk_reduce.restype = c_int
        _state["lib"] = lib
    return lib


def status_word(device) -> torch.Tensor:
    """The int32 word in which kernels of this process record a fault (0 = none)."""
    key = ("status", device)
    word = _state.get(key)
    if word is None:
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        word = _state.get(("status", device))
        if word is None:
            word = _state[("status", device)] = torch.zeros(1, dtype=torch.int32, device=device)
        _state[key] = word                                # the same word under every spelling of the device
    return word


def _num_sms(device) -> int:
    key = ("sms", device)
    if key not in _state:
        _state[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _state[key]


_plans: dict = {}


def plan(m: int, n: int, k: int, num_sms: int, deferred: bool = False):
    """(token-tile width, K splits) the kernel will use for this problem; `deferred`: for a caller
    that leaves the partial sums of a split K to the consumer kernel (a split is cheaper then)."""
    key = (m, n, k, num_sms, bool(deferred))
    p = _plans.get(key)
    if p is None:
        bn, splits = c_int(0), c_int(0)
        _lib().fl_gemm_tc_plan_for(m, n, k, num_sms, int(bool(deferred)), ctypes.byref(bn), ctypes.byref(splits))
        p = _plans[key] = (bn.value, splits.value)
    return p


SCRATCH = "split-K partial sums"


def _workspace(device, floats: int) -> torch.Tensor:
    """Float scratch for split-K partial sums (see `scratch`: grows on demand, never inside
    a graph capture, and a growth invalidates captured graphs)."""
    return scratch.get(device, SCRATCH, floats, at_least=4 << 20)


def workspace_floats(m: int, n: int, k: int, device) -> int:
    """Floats of scratch that the product [m, k] x [n, k]^T takes (0 when its plan has no K split)."""
    need = 0
    for deferred in (False, True):
        _, splits = plan(m, n, k, _num_sms(device), deferred)
        if splits > 1:
            need = max(need, splits * m * (-(-n // 4) * 4))
    return need


def reserve(device, n: int, k: int, max_tokens: int) -> None:
    """Size the scratch for every step of up to `max_tokens` tokens of an [n, k] weight.  Up to
    1024 tokens the plan weighs candidates by a cost model, so every count is asked; above that
    the splits depend on the number of token tiles only, and within a bracket of 64 tokens the
    largest need is at the bracket's top."""
    counts = list(range(1, min(1024, max_tokens) + 1)) + list(range(1088, max_tokens + 64, 64))
    need = max(workspace_floats(min(m, max_tokens), n, k, device) for m in counts)
    scratch.reserve(device, SCRATCH, need)


class PackedWeight:
    """A weight matrix [n, k] packed by k-block for the tensor-core kernels: [ceil(k / 64)][n][64], so
    that the 128 rows x 64 columns of a stage's tile are 16 KB in one piece (from the row-major
    matrix DRAM serves them 128 bytes at a time from 128 pages: streaming products are 4 to 7 %
    slower).  Made once, when a model is loaded; the kernels take either layout."""

    def __init__(self, weight: torch.Tensor):
        if weight.dtype != torch.bfloat16 or weight.dim() != 2 or (weight.shape[1] > 1 and weight.stride(1) != 1):
            raise ops.KernelError("only a bfloat16 matrix with a dense last axis can be packed")
        self.n, self.k = weight.shape
        self.shape = (self.n, self.k)
        self.dtype, self.device = weight.dtype, weight.device
        self.data = torch.empty((-(-self.k // 64), self.n, 64), dtype=torch.bfloat16, device=weight.device)
        rc = _lib().fl_pack_weight(ops._ptr(weight), ops._ld(weight), ops._ptr(self.data), self.n, self.k, ops._stream())
        ops._check(rc, "pack_weight")

    def data_ptr(self) -> int:
        return self.data.data_ptr()

    def unpacked(self) -> torch.Tensor:
        """The row-major matrix again (tests)."""
        return self.data.permute(1, 0, 2).reshape(self.n, -1)[:, :self.k].contiguous()


def _weight_args(w):
    """(pointer, leading dimension) of a weight for the kernels: a leading dimension of 0 says packed."""
    if isinstance(w, PackedWeight):
        return c_void_p(w.data_ptr()), 0
    ldw = ops._ld(w)
    if ldw % 8 or w.data_ptr() % 16:
        raise ops.KernelError("tensor-core gemm: operands must be 16-byte aligned with a row pitch "
                              "that is a multiple of 8 elements")
    return ops._ptr(w), ldw


class Partial:
    """A product left as split-K partial sums: `splits` float slabs [rows, ld] in
    the shared workspace, to be added (in slab order) by the kernel that reads
    them.  The workspace is reused by the next split-K product, so a Partial must
    be consumed before that; `check()` raises if it was not."""

    def __init__(self, data, splits, rows, cols, ld, device):
        self.data, self.splits, self.rows, self.cols, self.ld = data, splits, rows, cols, ld
        self.split_stride = rows * ld
        self.device = device
        self.serial = _state.get(("serial", device), 0)

    def check(self):
        if self.serial != _state.get(("serial", self.device), 0):
            raise RuntimeError("split-K partial sums were overwritten by a later product before use")

    def reduce_into(self, out: torch.Tensor) -> torch.Tensor:
        """out[rows, cols] = the slabs added in order: for consumers without a kernel of their
        own that adds them while reading."""
        self.check()
        if tuple(out.shape) != (self.rows, self.cols):
            raise ops.KernelError(f"reduce: partial sums are {(self.rows, self.cols)}, out is {tuple(out.shape)}")
        rc = _lib().fl_splitk_reduce(ops._ptr(self.data), self.ld, self.splits, ops._ptr(out),
                                     ops.dtype_code(out), ops._ld(out), self.rows, self.cols, ops._stream())
        ops._check(rc, "splitk_reduce")
        return out


_launches: dict = {}        # operands' places and sizes -> (launcher, converted arguments, ...): see gemm
_scratch_seen: dict = {}    # device -> the scratch generation the remembered launches belong to


def _forget_if_scratch_moved(device) -> None:
    """Remembered launches hold the scratch buffer's address (and the Partial handed out for it):
    none of them survives a buffer that was replaced."""
    gen = scratch.generation(device)
    if _scratch_seen.get(device) != gen:
        _launches.clear()
        _scratch_seen[device] = gen


def _remember(key, launch) -> None:
    """Only addresses and sizes are kept, no tensor (but the scratch buffer inside a Partial): memory
    that is freed and handed out again under a remembered address gets the same launch, rightly."""
    if len(_launches) > 8192:           # (a few hundred in practice: layers x products x step sizes met)
        _launches.clear()
    _launches[key] = launch


def gemm(a: torch.Tensor, w, out: torch.Tensor, bn: int = 0, splits: int = 0,
         defer: bool = False):
    """out[M, N] = a[M, K] @ w[N, K]^T; a and w bfloat16 (row pitch a multiple of 8
    elements, base 16-byte aligned; w may be a PackedWeight), out bfloat16 or float32.

    With `defer`, a product whose K is split returns a Partial instead of
    writing `out`: its consumer adds the slabs while it reads them."""
    # A product asked for again with the same operands in the same places (a layer's buffers do not move
    # from step to step) is launched from what the first call worked out: the checks, the plan and the
    # argument conversions below cost more host time than the driver's launch.
    _forget_if_scratch_moved(a.device)
    key = (a.data_ptr(), a.shape, a.stride(0), a.dtype, w.data_ptr(), w.shape, out.data_ptr(), out.shape,
           out.stride(0), out.dtype, bn, splits, defer)
    known = _launches.get(key)
    if known is not None:
        fn, args, kernels, partial = known
        if partial is not None:
            serial_key = ("serial", a.device)
            partial.serial = _state[serial_key] = _state.get(serial_key, 0) + 1
        elif kernels == 2:
            serial_key = ("serial", a.device)
            _state[serial_key] = _state.get(serial_key, 0) + 1
        ops._check(fn(*args, ops._stream()), "gemm_tcgen05", kernels)
        return partial
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ops.KernelError("tensor-core gemm takes bfloat16 operands")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise ops.KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if m == 0:
        return
    lda, ldc = ops._ld(a), ops._ld(out)
    if lda % 8 or a.data_ptr() % 16:
        raise ops.KernelError("tensor-core gemm: operands must be 16-byte aligned with a row pitch "
                              "that is a multiple of 8 elements")
    w_ptr, ldw = _weight_args(w)
    sms = _num_sms(a.device)
    if bn == 0:
        bn, splits = plan(m, n, k, sms, defer)
    ws, ws_floats = None, 0
    if splits > 1:
        ws_floats = splits * m * (-(-n // 4) * 4)
        ws = _workspace(a.device, ws_floats)
        ws_floats = ws.numel()
    deferred = defer and splits > 1
    fn = _lib().fl_gemm_tc_partial if deferred else _lib().fl_gemm_tc
    if splits > 1:
        serial_key = ("serial", a.device)
        _state[serial_key] = _state.get(serial_key, 0) + 1    # earlier Partials are now stale
    args = (ops._ptr(a), lda, w_ptr, ldw, ops._ptr(out), ops.dtype_code(out), ldc,
            m, n, k, bn, splits, ops._ptr(ws), ws_floats, sms, ops._ptr(status_word(a.device)))
    kernels = 2 if (splits > 1 and not deferred) else 1
    ops._check(fn(*args, ops._stream()), "gemm_tcgen05", kernels)
    partial = Partial(ws, splits, m, n, -(-n // 4) * 4, a.device) if deferred else None
    _remember(key, (fn, args, kernels, partial))
    return partial


def gemm_swiglu(a: torch.Tensor, w, out: torch.Tensor) -> bool:
    """out[M, I] = silu(a @ gate^T) * (a @ up^T) for w = [gate; up] stacked as [2 I, K], all
    bfloat16, in one kernel (the activation in the product's epilogue).  Returns False, having
    done nothing, when the kernel does not take the problem (its plan splits K)."""
    key = ("swiglu", a.data_ptr(), a.shape, a.stride(0), a.dtype, w.data_ptr(), w.shape, out.data_ptr(), out.shape,
           out.stride(0), out.dtype)
    known = _launches.get(key)                              # (see gemm)
    if known is not None:
        if known is False:
            return False
        ops._check(known[0](*known[1], ops._stream()), "gemm_tcgen05 (gated)")
        return True
    m, k = a.shape
    inter = w.shape[0] // 2
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16
            or w.shape[0] != 2 * inter or w.shape[1] != k or tuple(out.shape) != (m, inter)):
        raise ops.KernelError(f"gemm_swiglu: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}, "
                              f"{a.dtype}/{w.dtype}/{out.dtype}")
    if m == 0:
        return True
    lda = ops._ld(a)
    if lda % 8 or a.data_ptr() % 16:
        return False
    try:
        w_ptr, ldw = _weight_args(w)
    except ops.KernelError:
        return False
    fn = _lib().fl_gemm_tc_swiglu
    args = (ops._ptr(a), lda, w_ptr, ldw, ops._ptr(out), ops._ld(out), m, inter, k,
            _num_sms(a.device), ops._ptr(status_word(a.device)))
    rc = fn(*args, ops._stream())
    if rc == -1:
        _remember(key, False)
        return False
    ops._check(rc, "gemm_tcgen05 (gated)")
    _remember(key, (fn, args))
    return True


def gemm_qkv_rope(a: torch.Tensor, w, q_out: torch.Tensor, n_heads: int, n_kv_heads: int,
                  head_dim: int, rot_dim: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                  slots: torch.Tensor, cache: torch.Tensor, page_size: int) -> bool:
    """The q|k|v product of an attention layer with the rotary encoding and the cache write in its
    epilogue: q_out[M, n_heads * head_dim] gets the rotated queries, `cache`
    ([pages, 2, kv_heads, page_size, head_dim]) the rotated keys and the values at the tokens' `slots`;
    w = [q; k; v] stacked as [(n_heads + 2 n_kv_heads) * head_dim, K], all bfloat16.  Returns False,
    having done nothing, when the kernel does not take the problem (heads not of 128 rotated in full,
    64 tokens or fewer, a plan that splits K)."""
    key = ("qkv", a.data_ptr(), a.shape, a.stride(0), a.dtype, w.data_ptr(), w.shape, q_out.data_ptr(), q_out.shape,
           q_out.stride(0), q_out.dtype, n_heads, n_kv_heads, head_dim, rot_dim, cos.data_ptr(), sin.data_ptr(),
           cos.shape, positions.data_ptr(), slots.data_ptr(), cache.data_ptr(), cache.shape, cache.dtype, page_size)
    known = _launches.get(key)                              # (see gemm)
    if known is not None:
        if known is False:
            return False
        ops._check(known[0](*known[1], ops._stream()), "gemm_tcgen05 (q|k|v with rotary)")
        return True
    m, k = a.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16
            or cache.dtype != torch.bfloat16 or tuple(w.shape) != ((n_heads + 2 * n_kv_heads) * head_dim, k)
            or tuple(q_out.shape) != (m, n_heads * head_dim) or cos.dtype != torch.float32):
        raise ops.KernelError(f"gemm_qkv_rope: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(q_out.shape)}, "
                              f"{a.dtype}/{w.dtype}/{q_out.dtype}/{cache.dtype}")
    if m == 0:
        return True
    lda = ops._ld(a)
    if lda % 8 or a.data_ptr() % 16 or not cache.is_contiguous() \
            or cos.shape[1] * 2 != rot_dim or not cos.is_contiguous() or not sin.is_contiguous():
        return False
    try:
        w_ptr, ldw = _weight_args(w)
    except ops.KernelError:
        return False
    k_ptr = c_void_p(cache.data_ptr())
    v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
    fn = _lib().fl_gemm_tc_qkv_rope
    args = (ops._ptr(a), lda, w_ptr, ldw, ops._ptr(q_out), ops._ld(q_out), m, k,
            n_heads, n_kv_heads, head_dim, rot_dim, ops._ptr(positions), ops._ptr(slots),
            ops._ptr(cos), ops._ptr(sin), k_ptr, v_ptr, cache.stride(0), page_size,
            _num_sms(a.device), ops._ptr(status_word(a.device)))
    rc = fn(*args, ops._stream())
    if rc == -1:
        _remember(key, False)
        return False
    ops._check(rc, "gemm_tcgen05 (q|k|v with rotary)")
    _remember(key, (fn, args))
    return True


class TensorCoreLinear:
    """A weight made ready for the tensor-core kernels: packed by k-block (see PackedWeight), or, with
    `pack=False` (a matrix that something else reads row-major as well: a tied embedding table),
    left as it is, padded once if its row pitch is not a multiple of 16 bytes."""

    def __init__(self, weight: torch.Tensor, pack: bool = True):
        if pack:
            self.weight = PackedWeight(weight)
            return
        n, k = weight.shape
        if k % 8 or weight.data_ptr() % 16 or not weight.is_contiguous():
            pitch = -(-k // 8) * 8
            padded = torch.zeros((n, pitch), dtype=weight.dtype, device=weight.device)
            padded[:, :k] = weight
            weight = padded[:, :k]
        self.weight = weight

    def forward(self, a: torch.Tensor, out: torch.Tensor, defer: bool = False):
        return gemm(a, self.weight, out, defer=defer)
