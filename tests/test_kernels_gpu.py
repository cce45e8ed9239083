"""Each CUDA kernel alone against a plain torch float32 reference of the same
operation, at sizes other than the models' (odd widths, tails, many shapes)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


# ----------------------------------------------------------------------- GEMM

GEMM_SHAPES = [(1, 128, 64), (3, 96, 96), (7, 32, 172), (16, 320, 264), (17, 515, 200), (33, 130, 72),
               (64, 256, 1024), (100, 384, 328), (129, 640, 512), (300, 257, 136), (513, 128, 64)]


@pytest.mark.parametrize("m, n, k", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_gemm(m, n, k, out_dtype):
    from fastllm_py_b200.native import gemm_tc

    g = torch.Generator(device="cpu").manual_seed(m * 1000 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    pitch = -(-k // 8) * 8
    a_dev = torch.zeros(m, pitch, dtype=torch.bfloat16, device=DEV)
    a_dev[:, :k] = a.to(DEV)
    a_dev[:, k:] = 7.0                                # padding must never be read
    lin = gemm_tc.TensorCoreLinear(w.to(DEV))
    out = torch.full((m, n + 3), -5.0, dtype=out_dtype, device=DEV)
    lin.forward(a_dev[:, :k], out[:, :n])
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    got = out[:, :n].float().cpu()
    assert torch.all(out[:, n:] == -5.0), "wrote outside the output columns"
    tol = 1e-3 * math.sqrt(k) if out_dtype == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
    assert float((got - ref).abs().max()) <= tol


@pytest.mark.parametrize("bn, splits", [(16, 1), (16, 4), (32, 3), (64, 2), (128, 1), (128, 6), (256, 1), (256, 2), (16, 12)])
def test_tensor_core_gemm_every_tile_and_split(bn, splits):
    """Every tile width and split count, forced, against float32."""
    from fastllm_py_b200.native import gemm_tc

    m, n, k = min(bn, 200) + 5, 300, 64 * 11 + 24
    g = torch.Generator(device="cpu").manual_seed(bn + splits)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    gemm_tc.gemm(a.to(DEV), w.to(DEV), out, bn=bn, splits=splits)
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    assert float((out.cpu() - ref).abs().max()) <= 1e-3 * math.sqrt(k)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bn, splits, m", [(576, 1, 90), (576, 3, 33), (640, 1, 150), (640, 4, 261), (512, 1, 300),
                                           (512, 2, 517), (512, 6, 40)])
def test_tensor_core_gemm_in_cta_pairs_every_tile_and_split(bn, splits, m, out_dtype):
    """The CTA-pair kernel, forced, with token tiles of 64, 128 and 256 (codes 576, 640, 512), whole K and
    split K, token and feature counts that end inside a tile, an output pitch wider than the
    product and, for one case, an output that is not 16-byte aligned (its rows then leave one
    value at a time); and the same product left as partial sums."""
    from fastllm_py_b200.native import gemm_tc

    n, k = 300 + 256 * (splits % 2), 64 * 11 + 24
    g = torch.Generator(device="cpu").manual_seed(bn + splits + m)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    tol = 1e-3 * math.sqrt(k) if out_dtype == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
    for shift in (0, 1):
        pitch = n + 8 + shift                               # shift 1: rows no longer start on 16 bytes
        out = torch.full((m, pitch), -5.0, dtype=out_dtype, device=DEV)
        gemm_tc.gemm(a.to(DEV), w.to(DEV), out[:, shift:shift + n], bn=bn, splits=splits)
        torch.cuda.synchronize()
        assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
        assert torch.all(out[:, shift + n:] == -5.0) and torch.all(out[:, :shift] == -5.0), "wrote outside the output"
        assert float((out[:, shift:shift + n].float().cpu() - ref).abs().max()) <= tol
    if splits > 1:
        out = torch.full((m, n), -5.0, dtype=out_dtype, device=DEV)
        part = gemm_tc.gemm(a.to(DEV), w.to(DEV), out, bn=bn, splits=splits, defer=True)
        torch.cuda.synchronize()
        assert part is not None and part.splits == splits and torch.all(out == -5.0)
        slabs = part.data[:splits * part.split_stride].view(splits, m, part.ld)[:, :, :n]
        assert float((slabs.sum(0).cpu() - ref).abs().max()) <= 1e-3 * math.sqrt(k)


@pytest.mark.parametrize("m, n, k", [(3, 300, 728), (40, 130, 72), (70, 515, 200), (300, 700, 1000), (600, 257, 520)])
def test_packed_weights_give_the_row_major_result(m, n, k):
    """A weight packed by k-block ([ceil(K / 64)][N][64], what a model's matrices become at load) and
    the same weight row-major go through the same kernels and give the same result bit for bit: the
    plain product (one tile a CTA and CTA pairs, K whole and split, feature and K counts that end
    inside a tile) and the product with the SwiGLU epilogue."""
    from fastllm_py_b200.native import gemm_tc

    g = torch.Generator(device="cpu").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    pitch = -(-k // 8) * 8
    a_dev = torch.zeros(m, pitch, dtype=torch.bfloat16, device=DEV)[:, :k]
    a_dev.copy_(a)
    w_dev = torch.zeros(n, pitch, dtype=torch.bfloat16, device=DEV)[:, :k]
    w_dev.copy_(w)
    packed = gemm_tc.PackedWeight(w_dev)
    assert torch.equal(packed.unpacked().cpu(), w)
    outs = []
    for weight in (w_dev, packed):
        out = torch.full((m, n), -5.0, dtype=torch.float32, device=DEV)
        gemm_tc.gemm(a_dev, weight, out)
        outs.append(out.clone())
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    assert torch.equal(outs[0], outs[1])
    assert float((outs[1].cpu() - a.float() @ w.float().t()).abs().max()) <= 1e-3 * math.sqrt(k)
    if n % 2 == 0:
        acts = []
        for weight in (w_dev, packed):
            act = torch.full((m, n // 2), -5.0, dtype=torch.bfloat16, device=DEV)
            if not gemm_tc.gemm_swiglu(a_dev, weight, act):
                break
            acts.append(act.clone())
        if len(acts) == 2:
            assert torch.equal(acts[0], acts[1])


def test_tensor_core_gemm_plan_is_launchable():
    """What the plan answers for many problem sizes is a kernel the launcher has, with no empty split."""
    from fastllm_py_b200.native import gemm_tc

    for m in (1, 7, 64, 65, 128, 129, 300, 1000, 5000):
        for n, k in ((64, 64), (300, 1000), (4096, 4096), (12288, 4096), (4096, 11008), (102400, 4096)):
            bn, splits = gemm_tc.plan(m, n, k, 148)
            assert bn in (16, 32, 64, 128, 256, 512, 576, 640)
            kb = -(-k // 64)
            per = -(-kb // splits)
            assert 1 <= splits <= 16 and (splits - 1) * per < kb
            assert (bn <= 64) if m <= 64 else (bn >= 64)
            if m > 1024:
                assert bn == 512
            for deferred in (False, True):
                bn, splits = gemm_tc.plan(m, n, k, 148, deferred)
                assert bn in (16, 32, 64, 128, 256, 512, 640) and 1 <= splits <= 16
                assert (splits - 1) * -(-kb // splits) < kb


@pytest.mark.parametrize("a_dt, w_dt, c_dt", [(torch.float32, torch.float32, torch.float32),
                                              (torch.float32, torch.bfloat16, torch.float32),
                                              (torch.bfloat16, torch.float32, torch.bfloat16),
                                              (torch.bfloat16, torch.bfloat16, torch.float32)])
def test_cuda_core_gemm(a_dt, w_dt, c_dt):
    from fastllm_py_b200.native import ops

    for m, n, k in [(1, 7, 5), (5, 130, 172), (70, 65, 33), (129, 320, 264)]:
        a = torch.randn(m, k).to(a_dt)
        w = torch.randn(n, k).to(w_dt)
        ref = a.double() @ w.double().t()
        out = torch.zeros(m, n, dtype=c_dt, device=DEV)
        ops.gemm_simt(a.to(DEV), w.to(DEV), out)
        tol = 1e-5 * math.sqrt(k) * 4 if c_dt == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
        assert float((out.double().cpu() - ref).abs().max()) <= tol


# ------------------------------------------------------------------ attention

class AttentionCase:
    """Requests with cached context and new query tokens, their keys and values
    scattered over randomly chosen pages, plus a plain float reference."""

    def __init__(self, q_lens, ctx_lens, heads, kv_heads, head_dim, page_size, dtype, seed=0,
                 spikes=()):
        g = torch.Generator().manual_seed(seed)
        self.heads, self.kv_heads, self.head_dim, self.page_size = heads, kv_heads, head_dim, page_size
        self.q_lens, self.ctx_lens = q_lens, ctx_lens
        n = len(q_lens)
        totals = [c + q for c, q in zip(ctx_lens, q_lens)]
        pages_per = [-(-t // page_size) for t in totals]
        n_pages = sum(pages_per) + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.k_full = [torch.randn(t, kv_heads, head_dim, generator=g) for t in totals]
        self.v_full = [torch.randn(t, kv_heads, head_dim, generator=g) for t in totals]
        q_rows = [torch.randn(ql, heads, head_dim, generator=g) for ql in q_lens]
        # spikes: (request, query row, key position, query head): that key's score stands out
        for (r, row, key_pos, h) in spikes:
            direction = torch.randn(head_dim, generator=g)
            direction = direction / direction.norm()
            self.k_full[r][key_pos, h // (heads // kv_heads)] = direction * 12.0
            q_rows[r][row, h] = direction * 12.0
        rt = lambda x: x.to(dtype).to(torch.float32)            # what the device will hold
        self.k_full = [rt(k) for k in self.k_full]
        self.v_full = [rt(v) for v in self.v_full]
        q_rows = [rt(x) for x in q_rows]
        self.q_rows = q_rows
        cache = torch.zeros(n_pages, 2, kv_heads, page_size, head_dim)
        cache[:] = float("nan") if dtype == torch.float32 else 1e4   # unowned pages hold poison
        bt = torch.full((n, max(pages_per)), -1, dtype=torch.int32)
        at = 0
        for r in range(n):
            for lp in range(pages_per[r]):
                pg = perm[at]
                at += 1
                bt[r, lp] = pg
                lo, hi = lp * page_size, min((lp + 1) * page_size, totals[r])
                cache[pg, 0, :, :hi - lo] = self.k_full[r][lo:hi].transpose(0, 1)
                cache[pg, 1, :, :hi - lo] = self.v_full[r][lo:hi].transpose(0, 1)
                cache[pg, :, :, hi - lo:] = 0.0
        self.cache = cache.to(dtype).to(DEV)
        self.block_table = bt.to(DEV)
        self.q = torch.cat([x.reshape(x.shape[0], heads * head_dim) for x in q_rows]).to(dtype).to(DEV)
        starts = [0]
        for ql in q_lens:
            starts.append(starts[-1] + ql)
        self.n_tokens = starts[-1]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.req_start, self.req_ctx, self.req_qlen = i32(starts), i32(ctx_lens), i32(q_lens)
        self.tok_req = i32([r for r, ql in enumerate(q_lens) for _ in range(ql)])
        self.positions = i32([c + i for c, ql in zip(ctx_lens, q_lens) for i in range(ql)])
        self.decode_tokens = i32([starts[r] for r, ql in enumerate(q_lens) if ql == 1])
        self.dtype = dtype

    def reference(self, window=None):
        outs = []
        rep = self.heads // self.kv_heads
        for r, (ql, c) in enumerate(zip(self.q_lens, self.ctx_lens)):
            k = self.k_full[r].repeat_interleave(rep, dim=1)
            v = self.v_full[r].repeat_interleave(rep, dim=1)
            for i in range(ql):
                p = c + i
                lo = max(0, p - window + 1) if window else 0
                s = torch.einsum("hd,shd->hs", self.q_rows[r][i], k[lo:p + 1]) * self.head_dim ** -0.5
                w = torch.softmax(s.double(), dim=-1).float()
                outs.append(torch.einsum("hs,shd->hd", w, v[lo:p + 1]).reshape(-1))
        return torch.stack(outs)

    def tolerance(self):
        biggest = max(float(v.abs().max()) for v in self.v_full)
        return 1e-5 * biggest if self.dtype == torch.float32 else 2 ** -7 * biggest


def run_simt(case, window=None):
    from fastllm_py_b200.native import ops

    out = torch.zeros_like(case.q)
    ops.paged_attention_simt(case.q, out, case.cache, case.block_table, case.tok_req, case.positions,
                             case.heads, case.kv_heads, case.head_dim, window, case.head_dim ** -0.5,
                             case.page_size)
    return out.float().cpu()


def run_fast(case, window=None, prefill_variant=0, decode_variant=0, split_keys=256):
    from fastllm_py_b200.native import attention as fast

    out = torch.zeros_like(case.q)
    scale = case.head_dim ** -0.5
    n_dec = int(case.decode_tokens.numel())
    if n_dec:
        longest = max(c + q for c, q in zip(case.ctx_lens, case.q_lens) if q == 1)
        fast.decode_attention(case.q, out, case.cache, case.block_table, case.tok_req, case.positions,
                              None if n_dec == case.n_tokens else case.decode_tokens, n_dec, case.heads,
                              case.kv_heads, case.head_dim, window, scale, case.page_size,
                              fast.decode_splits(longest, split_keys), decode_variant, split_keys)
    if n_dec < case.n_tokens:
        fast.prefill_attention(case.q, out, case.cache, case.block_table, case.req_start, case.req_ctx,
                               case.req_qlen, len(case.q_lens), case.n_tokens, False, case.heads,
                               case.kv_heads, case.head_dim, window, scale, case.page_size, prefill_variant)
    return out.float().cpu()


ATT_SHAPES = [
    # q_lens, ctx_lens, heads, kv_heads, head_dim, page_size
    ([1, 1, 1], [0, 17, 300], 4, 4, 16, 16),
    ([5, 1, 33, 1], [0, 40, 7, 129], 6, 2, 48, 8),
    ([70, 2, 1], [0, 130, 600], 4, 2, 80, 32),
    ([130], [257], 8, 1, 128, 16),
    ([1, 1], [1023, 1024], 2, 2, 256, 64),
    ([64, 65, 63], [0, 64, 1], 3, 3, 112, 12),
]


@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37])
def test_cuda_core_attention(shape, dtype, window):
    case = AttentionCase(*shape, dtype, seed=1)
    diff = (run_simt(case, window) - case.reference(window)).abs().max()
    assert float(diff) <= case.tolerance()


@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
def test_tensor_core_and_split_key_attention(shape, window):
    case = AttentionCase(*shape, torch.bfloat16, seed=2)
    diff = (run_fast(case, window) - case.reference(window)).abs().max()
    assert float(diff) <= case.tolerance()


DECODE_SHAPES = [
    # q_lens, ctx_lens, heads, kv_heads, head_dim, page_size
    ([1, 1, 1], [0, 17, 300], 4, 4, 16, 16),
    ([1, 1], [1023, 1024], 2, 2, 256, 64),
    ([1, 1, 1, 1], [5, 255, 256, 700], 6, 2, 48, 8),          # three query heads per key/value head
    ([1, 1], [300, 1500], 8, 1, 128, 16),                     # eight
    ([1, 1, 1], [40, 511, 512], 32, 2, 64, 16),               # sixteen: the tensor-core kernel's most
    ([1], [333], 34, 2, 32, 16),                              # seventeen: the CUDA-core kernel serves it
    ([1, 1], [100, 200], 3, 3, 112, 12),                      # pages of 12 tokens
    ([1, 7, 1], [600, 3, 90], 4, 2, 80, 32),                  # decode tokens beside a prompt portion
]


@pytest.mark.parametrize("shape", DECODE_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 300])
@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("split_keys", [256, 64, 1024])
def test_decode_attention_both_kernels(shape, window, variant, split_keys):
    """variant 0: mma.sync over the heads of a group (where it applies); variant 1: CUDA cores;
    with the smallest split, the usual one and a large one."""
    case = AttentionCase(*shape, torch.bfloat16, seed=11)
    diff = (run_fast(case, window, 0, variant, split_keys) - case.reference(window)).abs().max()
    assert float(diff) <= case.tolerance()


TC_SHAPES = [
    # q_lens, ctx_lens, heads, kv_heads, head_dim, page_size: what the tcgen05 prefill kernel takes
    ([130], [257], 8, 1, 128, 16),
    ([5, 300, 128, 2], [0, 40, 7, 129], 6, 2, 64, 8),
    ([257, 1, 64], [0, 600, 1000], 4, 4, 128, 32),
    ([129, 127], [383, 0], 2, 2, 64, 128),
    ([700], [0], 3, 1, 128, 64),
]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
@pytest.mark.parametrize("variant", [1, 2])
def test_prefill_attention_both_tensor_core_kernels(shape, window, variant):
    """variant 1: mma.sync; variant 2: tcgen05 (S and P V in tensor memory)."""
    from fastllm_py_b200.native.gemm_tc import status_word

    case = AttentionCase(*shape, torch.bfloat16, seed=7)
    diff = (run_fast(case, window, variant) - case.reference(window)).abs().max()
    assert int(status_word(torch.device(DEV)).item()) == 0
    assert float(diff) <= case.tolerance()


def run_fast_tcgen05(case, window=None):
    return run_fast(case, window, 2)


def run_fast_cuda_core_decode(case, window=None):
    return run_fast(case, window, 0, 1)


@pytest.mark.parametrize("runner", [run_simt, run_fast, run_fast_tcgen05, run_fast_cuda_core_decode])
def test_a_far_key_among_hundreds_is_found(runner):
    """One key far back (and one right at a page edge, one at a split edge) gets
    nearly all the weight: the output must be that key's value."""
    ctx = 700
    spikes = [(0, 0, 3, 0), (0, 0, 15, 1), (0, 0, 16, 2), (0, 0, 255, 3), (0, 0, 256, 4),
              (0, 0, 511, 5), (1, 9, 64, 0), (1, 9, 63, 1), (1, 9, 700, 2), (1, 9, 0, 3)]
    case = AttentionCase([1, 10], [ctx, ctx], 6, 6, 64, 16, torch.bfloat16, seed=3, spikes=spikes)
    got = runner(case)
    ref = case.reference()
    assert float((got - ref).abs().max()) <= case.tolerance()
    for (r, row, key_pos, h) in spikes:
        t = row if r == 0 else 1 + row
        want = case.v_full[r][key_pos, h]
        assert float((got[t].reshape(6, 64)[h] - want).abs().max()) < 0.05, (r, row, key_pos, h)


@pytest.mark.parametrize("runner", [run_simt, run_fast, run_fast_cuda_core_decode])
def test_window_edge(runner):
    """A dominant key just outside the window must be ignored, one just inside must win."""
    window, ctx = 50, 300
    pos = ctx                                   # the single query token's position
    inside, outside = pos - window + 1, pos - window
    case = AttentionCase([1, 4], [ctx, ctx], 2, 2, 32, 16, torch.bfloat16, seed=4,
                         spikes=[(0, 0, outside, 0), (0, 0, inside, 1),
                                 (1, 3, ctx + 3 - window, 0), (1, 3, ctx + 3 - window + 1, 1)])
    got = runner(case, window)
    ref = case.reference(window)
    assert float((got - ref).abs().max()) <= case.tolerance()
    assert float((got[0].reshape(2, 32)[1] - case.v_full[0][inside, 1]).abs().max()) < 0.05
    assert float((got[0].reshape(2, 32)[0] - case.v_full[0][outside, 0]).abs().max()) > 0.5


# ------------------------------------------------ rotary + cache write, norms, SwiGLU

def rope_reference(x, pos, cos, sin, rot):
    """x: [T, heads, D] float; rotate-half over the first `rot` dimensions."""
    half = rot // 2
    x1, x2 = x[..., :half], x[..., half:rot]
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, head_dim, rot, page_size", [
    (4, 2, 16, 16, 8), (3, 3, 48, 48, 16), (8, 1, 128, 128, 16), (2, 2, 64, 32, 4), (5, 5, 80, 80, 12)])
def test_rope_and_cache_write(dtype, heads, kv_heads, head_dim, rot, page_size):
    """Every form of the kernel (scalar, 16-byte vectors, reading split-K partial
    sums) against a float reference, including partial rotation and odd pages."""
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.native.gemm_tc import Partial

    g = torch.Generator().manual_seed(head_dim + rot)
    n, n_pages, max_pos = 23, 9, 64
    cols = (heads + 2 * kv_heads) * head_dim
    store = (lambda t: t.to(dtype).float())
    qkv = store(torch.randn(n, cols, generator=g))
    pos = torch.randint(0, max_pos, (n,), generator=g)
    ang = torch.rand(max_pos, max(rot // 2, 1), generator=g) * 6.0
    cos, sin = torch.cos(ang), torch.sin(ang)
    slots = torch.randperm(n_pages * page_size, generator=g)[:n]
    slots[3] = -1                                                  # a token that must not be written
    q_ref = rope_reference(qkv[:, :heads * head_dim].reshape(n, heads, head_dim), pos, cos, sin, rot)
    k_ref = rope_reference(qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(n, kv_heads, head_dim),
                           pos, cos, sin, rot)
    v_ref = qkv[:, (heads + kv_heads) * head_dim:].reshape(n, kv_heads, head_dim)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7 * float(qkv.abs().max())
    dev = lambda t, dt=None: t.to(DEV if dt is None else DEV, dtype=dt) if dt else t.to(DEV)
    i32 = lambda t: t.to(torch.int32).to(DEV)

    def check(q_out, cache):
        cache = cache.float().cpu()
        assert float((q_out.float().cpu().reshape(n, heads, head_dim) - q_ref).abs().max()) <= tol
        for t in range(n):
            s = int(slots[t])
            if s < 0:
                continue
            pg, off = s // page_size, s % page_size
            assert float((cache[pg, 0, :, off] - k_ref[t]).abs().max()) <= tol
            assert float((cache[pg, 1, :, off] - v_ref[t]).abs().max()) <= tol
        written = {int(s) for s in slots if s >= 0}
        for s in range(n_pages * page_size):
            if s not in written:
                assert float(cache[s // page_size, :, :, s % page_size].abs().max()) == 0.0

    # in place on the activation buffer
    buf = qkv.to(dtype).to(DEV)
    cache = torch.zeros(n_pages, 2, kv_heads, page_size, head_dim, dtype=dtype, device=DEV)
    ops.rope_kv_write(buf, heads, kv_heads, head_dim, rot, cos.to(DEV), sin.to(DEV), i32(pos), i32(slots), cache,
                      page_size)
    check(buf[:, :heads * head_dim], cache)
    # from split-K partial sums: three slabs that add up to qkv
    if dtype == torch.bfloat16:
        ld = -(-cols // 4) * 4
        parts = torch.randn(3, n, ld, generator=g)
        parts[2, :, :cols] = qkv - parts[0, :, :cols] - parts[1, :, :cols]
        partial = Partial(parts.to(DEV).contiguous(), 3, n, cols, ld, torch.device(DEV))
        q_out = torch.zeros(n, heads * head_dim, dtype=dtype, device=DEV)
        cache2 = torch.zeros_like(cache)
        ops.rope_kv_write_partial(partial, q_out, heads, kv_heads, head_dim, rot, cos.to(DEV), sin.to(DEV),
                                  i32(pos), i32(slots), cache2, page_size)
        tol2 = tol + 2 ** -7 * float(qkv.abs().max())              # the sum is rounded once more on the way
        q_got = q_out.float().cpu().reshape(n, heads, head_dim)
        assert float((q_got - q_ref).abs().max()) <= tol2
        assert float((cache2.float() - cache.float()).abs().max()) <= tol2


@pytest.mark.parametrize("n", [5, 40])
@pytest.mark.parametrize("dim", [64, 70, 200, 1024, 1028, 4096, 5000, 9000])
def test_partial_sum_consumers(dim, n):
    """add+RMSNorm and SwiGLU reading split-K partial sums equal the same kernels on the summed input
    (rows of up to 8192 values in 16-byte chunks stay in registers; wider or odd ones go element by element)."""
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.native.gemm_tc import Partial

    g = torch.Generator().manual_seed(dim)
    splits = 4
    ld = -(-dim // 4) * 4
    parts = torch.randn(splits, n, ld, generator=g)
    total = parts[:, :, :dim].sum(0)
    partial = Partial(parts.to(DEV).contiguous(), splits, n, dim, ld, torch.device(DEV))
    resid = torch.randn(n, dim, generator=g)
    w = (1 + 0.1 * torch.randn(dim, generator=g)).to(torch.bfloat16)
    out = torch.zeros(n, dim, dtype=torch.bfloat16, device=DEV)
    r_dev = resid.clone().to(DEV)
    ops.add_rmsnorm_partial(r_dev, partial, w.to(DEV), out, 1e-6)
    delta = total.to(torch.bfloat16).float()
    want_resid = resid + delta
    want = want_resid * torch.rsqrt((want_resid ** 2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert float((r_dev.cpu() - want_resid).abs().max()) <= 2 ** -7 * float(total.abs().max())
    assert float((out.float().cpu() - want).abs().max()) <= 2 ** -6 * float(want.abs().max())
    if dim % 2 == 0:
        inter = dim // 2
        act = torch.zeros(n, inter, dtype=torch.bfloat16, device=DEV)
        ops.swiglu_partial(partial, act)
        gate, up = delta[:, :inter], delta[:, inter:dim]
        want = gate / (1 + torch.exp(-gate)) * up
        assert float((act.float().cpu() - want).abs().max()) <= 2 ** -7 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [8, 172, 11008, 77])
def test_swiglu_kernel(dtype, inter):
    from fastllm_py_b200.native import ops

    g = torch.Generator().manual_seed(inter)
    gu = (torch.randn(6, 2 * inter, generator=g) * 2).to(dtype)
    out = torch.zeros(6, inter, dtype=dtype, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    gf = gu.float()
    want = gf[:, :inter] / (1 + torch.exp(-gf[:, :inter])) * gf[:, inter:]
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7 * float(want.abs().max())
    assert float((out.float().cpu() - want).abs().max()) <= tol


def test_embedding_kernel_reports_bad_ids():
    from fastllm_py_b200.native import ops

    table = torch.randn(50, 72).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 50, 0, -1], dtype=torch.int32)
    out = torch.full((5, 72), 9.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(table.to(DEV), ids.to(DEV), out, status)
    got = out.cpu()
    assert torch.equal(got[[0, 1, 3]], table.float()[[3, 49, 0]])
    assert float(got[[2, 4]].abs().max()) == 0.0                # rows of ids outside the table are zeros
    assert int(status.item()) in (3, 5)                        # 1 + index of a bad id


@pytest.mark.parametrize("m", [1, 7, 16, 50, 100, 129, 300, 513])
@pytest.mark.parametrize("inter, k", [(11048, 320), (9728, 72), (13004, 136), (16648, 72), (5512, 264), (1380, 520)])
def test_gate_up_product_with_swiglu_epilogue(m, inter, k):
    """silu(a gate^T) * (a up^T) written by the product's epilogue (one-tile kernel for few
    tokens, with 16 to 64 features per CTA depending on the intermediate size; CTA pairs for
    many), against the product and the activation done apart; intermediate sizes that are no
    multiple of the tiles; nothing written outside."""
    from fastllm_py_b200.native import gemm_tc

    g = torch.Generator(device="cpu").manual_seed(m + inter + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    gu = (a.float() @ w.float().t()).to(torch.bfloat16).float()
    ref = gu[:, :inter] / (1.0 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    out = torch.full((m, inter + 5), -5.0, dtype=torch.bfloat16, device=DEV)
    done = gemm_tc.gemm_swiglu(a.to(DEV), w.to(DEV), out[:, :inter])
    if not done:                                                # many tokens, few features: the plan splits K
        assert m > 128 and inter < 9000, "this size should be taken by the fused kernel"
        torch.cuda.synchronize()
        assert torch.all(out == -5.0)
        return
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    assert torch.all(out[:, inter:] == -5.0), "wrote outside the output columns"
    got = out[:, :inter].float().cpu()
    # the factors may round to the neighbouring bfloat16 (another summation order), hence a few ulps
    tol = 2 ** -6 * float(ref.abs().max()) + 1e-3
    assert float((got - ref).abs().max()) <= tol


def test_gate_up_product_with_swiglu_epilogue_declines_split_problems():
    from fastllm_py_b200.native import gemm_tc

    a = torch.randn(4, 4096, device=DEV).to(torch.bfloat16)
    w = torch.randn(2 * 256, 4096, device=DEV).to(torch.bfloat16)      # few tiles: the plan splits K
    out = torch.full((4, 256), -5.0, dtype=torch.bfloat16, device=DEV)
    assert gemm_tc.gemm_swiglu(a, w, out) is False
    torch.cuda.synchronize()
    assert torch.all(out == -5.0)


# (the later shapes: token counts whose equally wide tiles are 96, 192, 160, 192 and 224 tokens wide)
@pytest.mark.parametrize("m, n, k", [(256, 256, 64), (300, 515, 200), (1024, 768, 1032), (257, 130, 72), (2048, 1024, 512),
                                     (97, 130, 72), (161, 515, 200), (385, 515, 200), (520, 300, 136), (673, 257, 72)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_gemm_cta_pairs(m, n, k, out_dtype):
    """The kernel in which two CTAs issue one 256 x 256 MMA together (cta_group::2), forced."""
    from fastllm_py_b200.native import gemm_tc

    g = torch.Generator(device="cpu").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    pitch = -(-k // 8) * 8
    a_dev = torch.zeros(m, pitch, dtype=torch.bfloat16, device=DEV)
    a_dev[:, :k] = a.to(DEV)
    lin = gemm_tc.TensorCoreLinear(w.to(DEV))
    out = torch.full((m, n + 3), -5.0, dtype=out_dtype, device=DEV)
    gemm_tc.gemm(a_dev[:, :k], lin.weight, out[:, :n], bn=512, splits=1)
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    assert torch.all(out[:, n:] == -5.0), "wrote outside the output columns"
    got = out[:, :n].float().cpu()
    tol = 1e-3 * math.sqrt(k) if out_dtype == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
    assert float((got - ref).abs().max()) <= tol
