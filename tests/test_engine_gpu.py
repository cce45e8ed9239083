"""The engine against the plain implementation, for every way of cutting the work.

Each tiny model runs the same requests whole, with the last 32 tokens one by
one, in portions of changing size (down to two tokens) and mixed (up to four
live requests, portions beside decoded tokens, a pool so small that pages are
used again), in true 32-bit and in bfloat16.  Every (request, position) is
compared with the plain whole-sequence logits.

Tolerances, fixed before the first run:
  * 32-bit vs plain: 1e-4 * max(1, largest |logit|);
  * 32-bit, one cut vs another: equal bit for bit (every kernel of that path
    sums in an order that depends on the token's own position only);
  * bfloat16 vs the plain implementation with bfloat16 storage emulated, request
    by request: twice the largest difference that bfloat16 storage itself makes
    to that request's plain logits, plus 1e-3; and at every position where the
    plain model's two best logits are further apart than twice the storage noise
    of that position (plus 1e-3), the engine's best token is the plain model's.

Every engine here runs with the cache's check mode on: pages that go back are
overwritten (and a fresh pool starts overwritten), so that a kernel that reads a
page its request no longer owns, or a place never written, shows in the logits.
The models are stored in bfloat16 and, for the 32-bit runs, also in float32 (all
products in float32 operands then).
"""
import numpy as np
import pytest
import torch

import plain_llama as plain
import replay
import tiny

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [5, 17, 33, 70, 100], "tiny_b": [1, 9, 40, 64, 100, 150],
           "tiny_c": [3, 47, 130, 64]}


def make_requests(name):
    cfg = tiny.CONFIGS[name]["config"]
    rng = np.random.default_rng(sum(map(ord, name)) + 1)
    return {f"r{i}": rng.integers(0, cfg.vocab_size, size=n).tolist()
            for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def plain_logits(name, folder, requests, bf16):
    key = (name, bf16, str(folder))
    if key not in _plain_cache:
        weights, config = plain.load_folder(folder)
        store = plain.store_bf16 if bf16 else plain.identity
        _plain_cache[key] = {rid: plain.forward(weights, config, toks, store=store)
                             for rid, toks in requests.items()}
    return _plain_cache[key]


_engines = {}


def engine_for(name, folder, dtype, max_tokens):
    from fastllm_py_b200 import Model

    key = (name, dtype, max_tokens, str(folder))
    if key not in _engines:
        page = tiny.CONFIGS[name]["page_size"]
        _engines[key] = Model.load(folder, dtype=dtype, page_size=page, max_tokens=max_tokens,
                                   max_requests=8, max_batched_tokens=512, max_model_len=256,
                                   cuda_graph=False, check_cache=True).engine
    return _engines[key]


class Tolerance:
    """What a cut's logits may differ by from the reference: one number (32-bit), or one per
    request plus the best-token rule (bfloat16)."""

    def __init__(self, overall=None, per_request=None, noise=None):
        self.overall, self.per_request, self.noise = overall, per_request, noise

    def of(self, rid):
        return self.overall if self.per_request is None else self.per_request[rid]

    def __float__(self):
        return float(self.overall if self.per_request is None else max(self.per_request.values()))


def tolerance(name, folder, requests, dtype):
    ref = plain_logits(name, folder, requests, dtype == "bfloat16")
    biggest = max(float(v.abs().max()) for v in ref.values())
    if dtype == "float32":
        return ref, Tolerance(1e-4 * max(1.0, biggest))
    exact = plain_logits(name, folder, requests, False)
    noise = {r: (ref[r] - exact[r]).abs().max(dim=1).values for r in ref}        # per position
    return ref, Tolerance(per_request={r: 2.0 * float(noise[r].max()) + 1e-3 for r in ref}, noise=noise)


def compare(got, ref, tol, what):
    assert got, "no logits came back"
    if not isinstance(tol, Tolerance):
        tol = Tolerance(float(tol))
    worst, where = 0.0, None
    for (rid, pos), row in got.items():
        d = float((row - ref[rid][pos]).abs().max()) / tol.of(rid)
        if not d <= worst:                      # also catches NaN
            worst, where = d, (rid, pos)
    assert worst <= 1.0, (f"{what}: largest difference {worst * tol.of(where[0]):.3e} at {where}, "
                          f"tolerance {tol.of(where[0]):.3e}")
    if tol.noise is not None:
        for (rid, pos), row in got.items():
            top2 = ref[rid][pos].topk(2).values
            if float(top2[0] - top2[1]) > 2.0 * float(tol.noise[rid][pos]) + 1e-3:
                assert int(row.argmax()) == int(ref[rid][pos].argmax()), \
                    f"{what}: another best token at {(rid, pos)} although the two best are {float(top2[0] - top2[1]):.3e} apart"


CUTS = {
    "whole": lambda reqs: replay.whole(reqs),
    "tail": lambda reqs: replay.tail_decode(reqs, 32),
    "portions": lambda reqs: replay.portions(reqs),
    "mixed": lambda reqs: replay.mixed(reqs, live=4, seed=3),
}


@pytest.fixture(scope="module")
def model_folders_f32(tmp_path_factory):
    """The tiny models stored in float32 (BASELINE's tiny-A and tiny-B are 32-bit models)."""
    root = tmp_path_factory.mktemp("models_f32")
    return {name: tiny.write(name, root / name, dtype="float32") for name in tiny.CONFIGS}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float32 stored in float32"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_cut_matches_plain(name, cut, dtype, model_folders, model_folders_f32):
    folders = model_folders
    if dtype.endswith("stored in float32"):
        dtype, folders = "float32", model_folders_f32
    requests = make_requests(name)
    steps = CUTS[cut](requests)
    ref, tol = tolerance(name, folders[name], requests, dtype)
    # the mixed cut gets a pool of exactly its peak, so that pages must be used again
    pool = replay.peak_tokens(steps) if cut == "mixed" else 512
    engine = engine_for(name, folders[name], dtype, pool)
    if folders is model_folders_f32:
        assert engine.decoder.blocks[0].mixer.qkv.weight.dtype == torch.float32
    poisoned = engine.cache.pages_poisoned
    got = replay.run_in_process(engine, steps)
    assert len(got) == sum(len(t) for t in requests.values())
    compare(got, ref, tol, f"{name} {cut} {dtype}")
    assert not engine.cache.live
    assert all(g.pool.free_pages == g.pool.num_pages for g in engine.cache.groups)
    assert engine.cache.pages_poisoned > poisoned            # the check mode was on: what went back was destroyed


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_float32_cuts_agree_bit_for_bit(name, model_folders):
    requests = make_requests(name)
    engine = engine_for(name, model_folders[name], "float32", 512)
    base = replay.run_in_process(engine, replay.whole(requests))
    for cut in ("tail", "portions", "mixed"):
        got = replay.run_in_process(engine, CUTS[cut](requests))
        for key, row in got.items():
            assert torch.equal(row, base[key]), f"{name} {cut}: {key} differs from the whole run"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, model_folders, tmp_path):
    """The program itself, as a subprocess, on a mixed trace with a tight pool."""
    name = "tiny_b"
    requests = make_requests(name)
    steps = replay.mixed(requests, live=4, seed=5)
    ref, tol = tolerance(name, model_folders[name], requests, dtype)
    vocab = tiny.CONFIGS[name]["config"].vocab_size
    got = replay.run_program(model_folders[name], dtype, steps, tmp_path / "out",
                             replay.peak_tokens(steps), vocab)
    compare(got, ref, tol, f"trace_run {dtype}")


def test_long_decoding(model_folders):
    """200 tokens decoded one by one after a short prompt, both precisions."""
    name = "tiny_b"
    cfg = tiny.CONFIGS[name]["config"]
    rng = np.random.default_rng(9)
    requests = {"long": rng.integers(0, cfg.vocab_size, size=230).tolist()}
    for dtype in ("float32", "bfloat16"):
        _plain_cache.clear()
        ref, tol = tolerance(name, model_folders[name], requests, dtype)
        engine = engine_for(name, model_folders[name], dtype, 512)
        got = replay.run_in_process(engine, replay.tail_decode(requests, 200))
        compare(got, ref, tol, f"long decoding {dtype}")
    _plain_cache.clear()


def test_decoding_together_across_changes_of_the_split(model_folders):
    """Three requests of different lengths decoded side by side for 450 steps with graph replay on:
    their lengths pass 256 and 512, where the decode kernel's keys per split (and with them the
    captured step) change, and one request ends on the way, which changes the batch."""
    from fastllm_py_b200 import Model
    from fastllm_py_b200.native.attention import decode_split_keys

    name = "tiny_c"
    cfg = tiny.CONFIGS[name]["config"]
    kv, hd = cfg.num_kv_heads, cfg.head_dim
    assert len({decode_split_keys(3, kv, n, 148, hd) for n in (200, 300, 600)}) > 1, "the choice never changes here"
    rng = np.random.default_rng(77)
    lengths = {"x": 640, "y": 520, "z": 470}
    requests = {r: rng.integers(0, cfg.vocab_size, size=n).tolist() for r, n in lengths.items()}
    weights, config = plain.load_folder(model_folders[name])
    ref = {r: plain.forward(weights, config, t, store=plain.store_bf16) for r, t in requests.items()}
    exact = {r: plain.forward(weights, config, t) for r, t in requests.items()}
    tol = 2.0 * max(float((ref[r] - exact[r]).abs().max()) for r in ref) + 1e-3
    model = Model.load(model_folders[name], dtype="bfloat16", page_size=tiny.CONFIGS[name]["page_size"],
                       max_tokens=2048, max_requests=4, max_batched_tokens=512, max_model_len=704,
                       cuda_graph=True)
    tail = 450
    steps = []
    for r, toks in requests.items():                        # the heads, one request a step
        steps.append({"step": len(steps), "end": [], "entries": [{"id": r, "tokens": toks[:len(toks) - tail], "want": []}]})
    for k in range(tail):                                   # then one token of each, together
        entries, end = [], []
        for r, toks in requests.items():
            at = len(toks) - tail + k
            if r == "z" and k >= 200:                       # z stops early
                continue
            entries.append({"id": r, "tokens": [toks[at]], "want": [0]})
            if k == tail - 1 or (r == "z" and k == 199):
                end.append(r)
        steps.append({"step": len(steps), "end": end, "entries": entries})
    got = replay.run_in_process(model.engine, steps)
    assert len(model.engine._graphs) >= 3
    compare(got, ref, tol, "decoding together across split changes")


def test_weights_stored_in_32_bit_stay_so(tmp_path):
    """A checkpoint stored in float32 run with bfloat16 activations: the matrices stay 32-bit
    (the CUDA-core product takes them), and the logits match the plain model."""
    import tiny as tiny_configs

    name = "tiny_a"
    folder = tiny_configs.write(name, tmp_path / "f32model", dtype="float32")
    from safetensors.torch import load_file
    assert load_file(str(folder / "model.safetensors"))["model.norm.weight"].dtype == torch.float32
    requests = make_requests(name)
    weights, config = plain.load_folder(folder)
    ref = {r: plain.forward(weights, config, t, store=plain.store_bf16) for r, t in requests.items()}
    exact = {r: plain.forward(weights, config, t) for r, t in requests.items()}
    tol = 2.0 * max(float((ref[r] - exact[r]).abs().max()) for r in ref) + 1e-3
    from fastllm_py_b200 import Model
    model = Model.load(folder, dtype="bfloat16", page_size=16, max_tokens=512, max_requests=8,
                       max_batched_tokens=512, max_model_len=256, cuda_graph=False)
    lin = model.decoder.blocks[0].mixer.qkv
    assert lin.weight.dtype == torch.float32
    got = replay.run_in_process(model.engine, replay.mixed(requests, live=3, seed=1))
    compare(got, ref, tol, "float32 weights under bfloat16 activations")


def test_wide_feed_forward_takes_the_fused_gate_up_kernels(tmp_path):
    """An intermediate size large enough that the gate|up product is planned without a K split:
    prompts then go through the CTA-pair kernel with the SwiGLU epilogue, decode steps through
    the one-tile kernel with it; compared in every cut with the plain implementation."""
    from fastllm_py_b200.config import LlamaConfig
    from fastllm_py_b200.native import gemm_tc
    from fastllm_py_b200.weights import write_model_folder
    from fastllm_py_b200 import Model

    cfg = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden_size=256, num_heads=2,
                      num_kv_heads=1, head_dim=128, intermediate_size=9640, vocab_size=1000,
                      rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
                      max_position_embeddings=1024, tie_word_embeddings=True)
    for m in (1, 4, 300):
        assert gemm_tc.plan(m, 2 * cfg.intermediate_size, cfg.hidden_size, 148)[1] == 1
    folder = write_model_folder(cfg, tmp_path / "wide", seed=8, std=0.03, norm_std=0.05)
    rng = np.random.default_rng(21)
    requests = {"w0": rng.integers(0, 1000, size=330).tolist(), "w1": rng.integers(0, 1000, size=90).tolist()}
    weights, config = plain.load_folder(folder)
    ref = {r: plain.forward(weights, config, t, store=plain.store_bf16) for r, t in requests.items()}
    exact = {r: plain.forward(weights, config, t) for r, t in requests.items()}
    tol = 2.0 * max(float((ref[r] - exact[r]).abs().max()) for r in ref) + 1e-3
    model = Model.load(folder, dtype="bfloat16", page_size=16, max_tokens=1024, max_requests=4,
                       max_batched_tokens=512, max_model_len=512, cuda_graph=False)
    for cut in ("whole", "tail", "portions", "mixed"):
        got = replay.run_in_process(model.engine, CUTS[cut](requests))
        compare(got, ref, tol, f"wide {cut}")


def test_medium_model_reaches_the_large_shape_kernels(tmp_path):
    """A model with head size 128, grouped heads and widths in the hundreds, so that whole prompts of
    several hundred tokens go through the persistent tensor-core product and the tcgen05 attention,
    decode steps through the split-K products whose partial sums the next kernel adds, in both cuts."""
    from fastllm_py_b200.config import LlamaConfig
    from fastllm_py_b200.weights import write_model_folder
    from fastllm_py_b200 import Model

    cfg = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden_size=512, num_heads=4,
                      num_kv_heads=2, head_dim=128, intermediate_size=1376, vocab_size=2000,
                      rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-6,
                      max_position_embeddings=1024, tie_word_embeddings=False)
    folder = write_model_folder(cfg, tmp_path / "medium", seed=3, std=0.03, norm_std=0.05)
    rng = np.random.default_rng(12)
    requests = {"m0": rng.integers(0, 2000, size=300).tolist(), "m1": rng.integers(0, 2000, size=70).tolist(),
                "m2": rng.integers(0, 2000, size=520).tolist()}
    weights, config = plain.load_folder(folder)
    ref = {r: plain.forward(weights, config, t, store=plain.store_bf16) for r, t in requests.items()}
    exact = {r: plain.forward(weights, config, t) for r, t in requests.items()}
    tol = 2.0 * max(float((ref[r] - exact[r]).abs().max()) for r in ref) + 1e-3
    model = Model.load(folder, dtype="bfloat16", page_size=16, max_tokens=2048, max_requests=4,
                       max_batched_tokens=1024, max_model_len=1024, cuda_graph=False)
    for cut in ("whole", "tail", "portions", "mixed"):
        steps = CUTS[cut](requests)
        got = replay.run_in_process(model.engine, steps)
        compare(got, ref, tol, f"medium {cut}")
    # the 32-bit path of the same model against the plain 32-bit logits
    model32 = Model.load(folder, dtype="float32", page_size=16, max_tokens=2048, max_requests=4,
                         max_batched_tokens=1024, max_model_len=1024, cuda_graph=False)
    biggest = max(float(v.abs().max()) for v in exact.values())
    got = replay.run_in_process(model32.engine, replay.portions(requests))
    compare(got, exact, 1e-4 * max(1.0, biggest), "medium float32")
