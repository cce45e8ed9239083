"""The kernels and the engine at the layer sizes that are timed (DeepSeek-LLM-7B: width 4096,
32 heads of 128, feed-forward 11008, vocabulary 102400), checked for values.

The small-size tests give a CTA pair of the tensor-core product one tile at most; here a pair
walks three tiles and more (the accumulator buffers wrap, the tile order has a second and a
short last panel), the decode attention runs the key splits the host picks at 2048 to 2304
keys, and the prompt attention runs 2048 rows of 32 heads.  Operands are random bfloat16 made
on the device; the reference is a plain float32 torch computation of sampled rows (all columns),
which is what fastllm-py's `verify()` does for its fast path at the size it ships
(fastllm_py/graph_decode.py:994-1032).
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _randn(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=DEV) * scale).to(torch.bfloat16)


def _status():
    from fastllm_py_b200.native.gemm_tc import status_word

    return int(status_word(torch.device(DEV)).item())


def _sample_rows(m, count=64, seed=0):
    """Rows spread over every token tile: the first and last of the product and random ones between."""
    rng = np.random.default_rng(seed)
    rows = sorted(set([0, 1, m - 1, m - 2, 255, 256, min(m - 1, 2047), min(m - 1, 2048)]
                      + rng.integers(0, m, size=count).tolist()))
    return torch.tensor(rows, device=DEV)


# ------------------------------------------------------------- tensor-core products

@pytest.mark.parametrize("n, k", [(4096, 4096), (12288, 4096), (4096, 11008)])
@pytest.mark.parametrize("m", [2048, 2304, 4160])
def test_pair_gemm_walks_many_tiles_and_panels(m, n, k):
    """The CTA-pair kernel as the plan launches it for a prompt step: 74 pairs over (n / 256) x
    ceil(m / 256) tiles is 2 to 11 tiles a pair; 2304 and 4160 tokens give the tile order a
    second panel of one and a short last panel."""
    from fastllm_py_b200.native import gemm_tc

    bn, splits = gemm_tc.plan(m, n, k, 148)
    assert bn == 512                                                     # the pair kernel, 256 tokens wide
    tiles = (n // 256) * -(-m // 256)
    assert tiles * splits >= 3 * 74 or splits > 1 or tiles > 74
    a, w = _randn((m, k), m + n), _randn((n, k), k + n + 1)
    out = torch.full((m, n), -5.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm(a, w, out)
    torch.cuda.synchronize()
    assert _status() == 0
    rows = _sample_rows(m, seed=m + k)
    ref = a[rows].float() @ w.float().t()
    tol = 2 ** -8 * float(ref.abs().max()) + 1e-3
    assert float((out[rows].float() - ref).abs().max()) <= tol
    # every element was written, and with something of the right size (no tile skipped, none doubled)
    assert float(out.float().abs().max()) <= 1.2 * float(ref.abs().max()) + 8 * math.sqrt(k)
    col_check = out.float().pow(2).mean(dim=0)                           # per feature, over all tokens
    assert float(col_check.min()) > 0.25 * k and float(col_check.max()) < 4.0 * k


@pytest.mark.parametrize("m", [2048, 2304])
def test_gated_pair_gemm_at_feed_forward_size(m):
    """gate|up product with the SwiGLU epilogue at 4096 -> 11008: 86 feature tiles x 8 or 9 token tiles."""
    from fastllm_py_b200.native import gemm_tc

    inter, k = 11008, 4096
    a, w = _randn((m, k), 3, 0.5), _randn((2 * inter, k), 4, 0.02)
    out = torch.full((m, inter), -5.0, dtype=torch.bfloat16, device=DEV)
    assert gemm_tc.gemm_swiglu(a, w, out)
    torch.cuda.synchronize()
    assert _status() == 0
    rows = _sample_rows(m, seed=5)
    g = (a[rows].float() @ w[:inter].float().t()).to(torch.bfloat16).float()
    u = (a[rows].float() @ w[inter:].float().t()).to(torch.bfloat16).float()
    ref = g / (1.0 + torch.exp(-g)) * u
    tol = 2 ** -7 * float(ref.abs().max()) + 1e-3
    assert float((out[rows].float() - ref).abs().max()) <= tol
    assert float(out.float().abs().max()) <= 1.5 * float(ref.abs().max()) + 1.0


@pytest.mark.parametrize("m", [8, 64])
def test_vocabulary_product_at_full_size(m):
    """The LM head of a decode step: 102400 features, float32 logits, the one-tile kernel."""
    from fastllm_py_b200.native import gemm_tc

    n, k = 102400, 4096
    a, w = _randn((m, k), 9), _randn((n, k), 10, 0.05)
    out = torch.full((m, n), -5.0, dtype=torch.float32, device=DEV)
    gemm_tc.gemm(a, w, out)
    torch.cuda.synchronize()
    assert _status() == 0
    ref = a.float() @ w.float().t()
    assert float((out - ref).abs().max()) <= 1e-3 * math.sqrt(k) * 0.05 * 4 + 1e-3
    assert torch.equal(out.argmax(dim=1), ref.argmax(dim=1)) or \
        float((ref.max(dim=1).values - ref.gather(1, out.argmax(dim=1)[:, None])[:, 0]).max()) < 1e-2


@pytest.mark.parametrize("m", [128, 256, 512, 768])
@pytest.mark.parametrize("n, k", [(4096, 4096), (4096, 11008), (12288, 4096)])
def test_products_of_prompt_portions(m, n, k):
    """Steps of a few hundred tokens: the plan's narrower tiles and K splits at the sizes it picks them for."""
    from fastllm_py_b200.native import gemm_tc

    a, w = _randn((m, k), m + 1), _randn((n, k), n + k)
    out = torch.full((m, n), -5.0, dtype=torch.bfloat16, device=DEV)
    part = gemm_tc.gemm(a, w, out, defer=True)
    if part is not None:
        part.reduce_into(out)
    torch.cuda.synchronize()
    assert _status() == 0
    ref = a.float() @ w.float().t()
    assert float((out.float() - ref).abs().max()) <= 2 ** -8 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("m", [128, 300, 520, 2304])
def test_qkv_product_with_rotary_and_cache_write_in_its_epilogue(m):
    """The q|k|v product at 4096 -> 12288 with heads of 128: the fused kernel (rotation and cache write in
    the product's epilogue) against the product followed by the rotary kernel, on the same inputs: the
    rotated queries and what lands in the cache pages are the same bit for bit, and pages of no token
    stay untouched.  At 300 tokens the cost model prefers the one-tile kernel followed by the rotary
    kernel (three token tiles of 128 fill one round of CTAs, two of 160 leave half the pairs a second
    tile): the fused call must then say so and touch nothing."""
    from fastllm_py_b200.native import gemm_tc, ops

    heads = kv_heads = 32
    k, hd, page = 4096, 128, 16
    a, w = _randn((m, k), m + 7, 0.5), _randn(((heads + 2 * kv_heads) * hd, k), 11, 0.05)
    g = torch.Generator().manual_seed(m)
    n_pages = -(-m // page) + 9
    perm = torch.randperm(n_pages, generator=g)[:-(-m // page)]
    positions = torch.arange(100, 100 + m, dtype=torch.int32)
    slots = (perm[torch.arange(m) // page] * page + torch.arange(m) % page).to(torch.int32)
    slots[5] = -1                                            # a token without a cache slot writes nothing
    ang = torch.arange(100 + m + 1, dtype=torch.float32)[:, None] * (10000.0 ** (-torch.arange(0, hd, 2) / hd))[None, :]
    cos, sin = torch.cos(ang).to(DEV).contiguous(), torch.sin(ang).to(DEV).contiguous()
    positions, slots = positions.to(DEV), slots.to(DEV)

    packed = gemm_tc.PackedWeight(w)

    def run(fused):
        cache = torch.full((n_pages, 2, kv_heads, page, hd), 3.0, dtype=torch.bfloat16, device=DEV)
        qkv = torch.full((m, (heads + 2 * kv_heads) * hd), -5.0, dtype=torch.bfloat16, device=DEV)
        if fused:
            took = gemm_tc.gemm_qkv_rope(a, packed if fused == "packed" else w, qkv[:, :heads * hd], heads, kv_heads,
                                         hd, hd, cos, sin, positions, slots, cache, page)
            assert took == (m != 300)
            if not took:
                torch.cuda.synchronize()
                assert bool((qkv == -5.0).all()) and bool((cache == 3.0).all())
                return None, None
        else:
            gemm_tc.gemm(a, w, qkv)
            ops.rope_kv_write(qkv, heads, kv_heads, hd, hd, cos, sin, positions, slots, cache, page)
        torch.cuda.synchronize()
        assert _status() == 0
        return qkv[:, :heads * hd].clone(), cache

    q_ref, cache_ref = run(False)
    for fused in (True, "packed"):                           # the weights row-major, and packed by k-block
        q_got, cache_got = run(fused)
        if q_got is None:
            return
        assert torch.equal(q_got, q_ref)
        assert torch.equal(cache_got, cache_ref)
    untouched = torch.ones(n_pages, dtype=torch.bool)
    untouched[perm] = False
    assert bool((cache_got[untouched.to(DEV)] == 3.0).all())


# ------------------------------------------------------------------------ attention

class PagedCase:
    """Requests whose keys and values sit in randomly chosen pages of a device cache
    [pages, 2, kv_heads, page_size, head_dim], with a float32 torch reference of chosen
    (request, query row, head) triples read back through the block table."""

    def __init__(self, q_lens, ctx_lens, heads, kv_heads, head_dim, page_size, seed):
        self.q_lens, self.ctx_lens = q_lens, ctx_lens
        self.heads, self.kv_heads, self.head_dim, self.page_size = heads, kv_heads, head_dim, page_size
        totals = [c + q for c, q in zip(ctx_lens, q_lens)]
        pages_per = [-(-t // page_size) for t in totals]
        n_pages = sum(pages_per) + 5
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(n_pages, generator=g)
        self.cache = _randn((n_pages, 2, kv_heads, page_size, head_dim), seed + 1)
        bt = torch.full((len(q_lens), max(pages_per)), -1, dtype=torch.int32)
        at = 0
        for r, p in enumerate(pages_per):
            bt[r, :p] = perm[at:at + p].to(torch.int32)
            at += p
        self.block_table = bt.to(DEV)
        self.n_tokens = sum(q_lens)
        self.q = _randn((self.n_tokens, heads * head_dim), seed + 2)
        starts = np.concatenate([[0], np.cumsum(q_lens)]).tolist()
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.starts = starts
        self.req_start, self.req_ctx, self.req_qlen = i32(starts), i32(ctx_lens), i32(q_lens)
        self.tok_req = i32([r for r, ql in enumerate(q_lens) for _ in range(ql)])
        self.positions = i32([c + i for c, ql in zip(ctx_lens, q_lens) for i in range(ql)])

    def spike(self, r, row, key_pos, head):
        """Make one far key stand out for one query: its output must then be that key's value."""
        g = torch.Generator(device=DEV).manual_seed(r * 7919 + row * 31 + key_pos + head)
        d = torch.randn(self.head_dim, generator=g, device=DEV)
        d = (d / d.norm() * 14.0).to(torch.bfloat16)
        page = int(self.block_table[r, key_pos // self.page_size])
        self.cache[page, 0, head // (self.heads // self.kv_heads), key_pos % self.page_size] = d
        self.q[self.starts[r] + row, head * self.head_dim:(head + 1) * self.head_dim] = d

    def reference(self, r, row, head):
        pos = self.ctx_lens[r] + row
        kvh = head // (self.heads // self.kv_heads)
        idx = torch.arange(pos + 1, device=DEV)
        pages = self.block_table[r, idx // self.page_size].long()
        k = self.cache[pages, 0, kvh, idx % self.page_size].float()
        v = self.cache[pages, 1, kvh, idx % self.page_size].float()
        q = self.q[self.starts[r] + row, head * self.head_dim:(head + 1) * self.head_dim].float()
        w = torch.softmax((k @ q).double() * self.head_dim ** -0.5, dim=0).float()
        return w @ v

    def check(self, out, triples, tol):
        worst = 0.0
        for (r, row, head) in triples:
            got = out[self.starts[r] + row, head * self.head_dim:(head + 1) * self.head_dim].float()
            worst = max(worst, float((got - self.reference(r, row, head)).abs().max()))
        assert worst <= tol, f"largest difference {worst:.3e}, tolerance {tol:.3e}"


@pytest.mark.parametrize("batch", [1, 8, 64])
def test_decode_attention_at_bench_shape(batch):
    """Single tokens of `batch` requests with 2048 to 2304 keys, 32 heads of 128 (MHA), pages of
    16, at the keys-per-split that the host picks for the launch (and two it does not)."""
    from fastllm_py_b200.native import attention as fast

    rng = np.random.default_rng(batch)
    ctx = [2047, 2303][:batch] + rng.integers(2048, 2304, size=max(0, batch - 2)).tolist()
    case = PagedCase([1] * batch, ctx, 32, 32, 128, 16, seed=100 + batch)
    case.spike(0, 0, 3, 5)                                   # a far key, first page
    case.spike(0, 0, 1023, 6)                                # last key of a 1024 split
    case.spike(batch - 1, 0, 768, 7)                         # first key of a 768 split
    picked = fast.decode_split_keys(batch, 32, max(ctx) + 1, 148, 128)
    triples = [(r, 0, h) for r in sorted({0, batch - 1, batch // 2}) for h in (0, 5, 6, 7, 31)]
    for keys in sorted({picked, 768, 1024}):
        out = torch.full_like(case.q, 7.0)
        fast.decode_attention(case.q, out, case.cache, case.block_table, case.tok_req, case.positions, None,
                              batch, 32, 32, 128, None, 128 ** -0.5, 16,
                              fast.decode_splits(max(ctx) + 1, keys), 0, keys)
        torch.cuda.synchronize()
        assert float(out.float().abs().max()) < 6.0          # every (token, head) was written
        case.check(out, triples, 2 ** -7 * 4.0)


def test_prompt_attention_at_bench_shape():
    """A 2048-token prompt (and a 300-token portion over 2000 cached keys) of 32 heads of 128
    on the tcgen05 kernel: 16 query tiles a head, up to 19 key blocks a tile."""
    from fastllm_py_b200.native import attention as fast

    case = PagedCase([2048, 300], [0, 2000], 32, 32, 128, 16, seed=77)
    case.spike(0, 2047, 0, 3)
    case.spike(0, 1500, 127, 4)
    case.spike(0, 1500, 128, 9)
    case.spike(1, 299, 17, 30)
    out = torch.full_like(case.q, 7.0)
    fast.prefill_attention(case.q, out, case.cache, case.block_table, case.req_start, case.req_ctx,
                           case.req_qlen, 2, case.n_tokens, False, 32, 32, 128, None, 128 ** -0.5, 16, 2)
    torch.cuda.synchronize()
    assert _status() == 0
    assert float(out.float().abs().max()) < 6.0
    rng = np.random.default_rng(3)
    triples = [(0, 2047, 3), (0, 1500, 4), (0, 1500, 9), (1, 299, 30), (0, 0, 0), (0, 127, 31), (0, 128, 1)]
    triples += [(0, int(rng.integers(0, 2048)), int(rng.integers(0, 32))) for _ in range(24)]
    triples += [(1, int(rng.integers(0, 300)), int(rng.integers(0, 32))) for _ in range(8)]
    case.check(out, triples, 2 ** -7 * 4.0)


# --------------------------------------------------------------------------- engine

def test_two_full_width_layers_bfloat16_against_float32(tmp_path):
    """Two layers at DeepSeek-LLM-7B width through the engine: a 2304-token prompt whole and in
    portions of 512, then 8 decode steps of a batch of 8, the bfloat16 path (tensor-core kernels,
    partial sums, fused epilogues, graph replay) against the true 32-bit path over the same
    weights, and the 32-bit path against the plain implementation on one 300-token request.

    Tolerance, by the rule of the tiny models' tests and fixed the same way: twice the largest
    difference that bfloat16 storage itself makes to the plain model's logits (measured on the
    300-token request) plus 1e-3; and the two paths' best tokens agree wherever the 32-bit
    path's two best are further apart than twice that."""
    import plain_llama as plain
    from fastllm_py_b200 import LlamaConfig, Model, StepEntry
    from fastllm_py_b200.weights import write_model_folder

    cfg = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden_size=4096, num_heads=32,
                      num_kv_heads=32, head_dim=128, intermediate_size=11008, vocab_size=3000,
                      rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-6,
                      max_position_embeddings=4096, tie_word_embeddings=False)
    folder = write_model_folder(cfg, tmp_path / "wide2", seed=3, std=0.02, norm_std=0.02)
    rng = np.random.default_rng(12)
    prompt = rng.integers(0, cfg.vocab_size, 2304).tolist()
    others = [rng.integers(0, cfg.vocab_size, 300 + 40 * i).tolist() for i in range(7)]
    decode = rng.integers(0, cfg.vocab_size, (8, 8)).tolist()
    want_rows = [0, 1, 255, 256, 511, 512, 1023, 2047, 2048, 2302, 2303]

    weights, config = plain.load_folder(folder)
    plain_exact = plain.forward(weights, config, others[0])
    plain_bf16 = plain.forward(weights, config, others[0], store=plain.store_bf16)
    del weights
    noise = float((plain_bf16 - plain_exact).abs().max())
    tol = 2.0 * noise + 1e-3

    def run(dtype, portions):
        model = Model.load(folder, dtype=dtype, page_size=16, max_tokens=8 * 2400, max_requests=8,
                           max_batched_tokens=2304, max_model_len=2400, cuda_graph=True)
        eng = model.engine
        got = []
        eng.begin("p")
        if portions:
            for at in range(0, 2304, 512):
                n = min(512, 2304 - at)
                want = [r - at for r in want_rows if at <= r < at + n]
                got.append(eng.step([StepEntry("p", prompt[at:at + n], want)]).to("cpu", copy=True))
        else:
            got.append(eng.step([StepEntry("p", prompt, want_rows)]).to("cpu", copy=True))
        first = None
        for i, o in enumerate(others):
            eng.begin(i)
            rows = eng.step([StepEntry(i, o, list(range(len(o))) if i == 0 else [])])
            if i == 0:
                first = rows.to("cpu", copy=True)
        rids = ["p"] + list(range(7))
        for k in range(8):
            got.append(eng.step([StepEntry(r, [decode[k][j]], [0]) for j, r in enumerate(rids)]).to("cpu", copy=True))
        eng.check_status()
        for r in rids:
            eng.end(r)
        eng.cache.check()
        del model
        torch.cuda.empty_cache()
        return torch.cat(got), first

    exact, first = run("float32", False)
    biggest = float(plain_exact.abs().max())
    assert float((first - plain_exact).abs().max()) <= 1e-4 * max(1.0, biggest), "the 32-bit path at full width"
    for portions in (False, True):
        got, first = run("bfloat16", portions)
        assert got.shape == exact.shape == (len(want_rows) + 64, cfg.vocab_size)
        assert float((first - plain_bf16).abs().max()) <= tol
        diff = (got - exact).abs().max(dim=1).values
        worst = int(diff.argmax())
        assert float(diff[worst]) <= tol, \
            f"portions={portions}: row {worst} differs by {float(diff[worst]):.3e}, tolerance {tol:.3e}"
        top2 = exact.topk(2, dim=1).values
        clear = (top2[:, 0] - top2[:, 1]) > 2 * tol
        assert bool((got.argmax(dim=1)[clear] == exact.argmax(dim=1)[clear]).all())
