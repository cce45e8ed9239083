"""Generation through the Python entry point and the scheduler, and the sampler on the device."""
import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
_models = {}


def model_for(name, folder, dtype, **opts):
    from fastllm_py_b200 import Model

    key = (name, dtype, tuple(sorted(opts.items())))
    if key not in _models:
        page = tiny.CONFIGS[name]["page_size"]
        base = dict(page_size=page, max_tokens=1024, max_requests=8, max_batched_tokens=64,
                    max_model_len=256)
        base.update(opts)
        _models[key] = Model.load(folder, dtype=dtype, **base)
    return _models[key]


def prompts_of(name, lengths, seed=4):
    cfg = tiny.CONFIGS[name]["config"]
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lengths]


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_matches_plain_float32(name, model_folders):
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "float32")
    for prompt in prompts_of(name, [5, 17, 33]):
        want = plain.generate(weights, config, prompt, 16)
        assert model.generate(prompt, max_new_tokens=16) == want
        assert model.generate(prompt, max_new_tokens=16, use_graph=False) == want


def test_greedy_generation_bfloat16(model_folders):
    """bfloat16 greedy follows the plain bfloat16-storage model; where the two part
    ways the plain model's two best logits must be nearly tied."""
    name = "tiny_c"
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "bfloat16")
    for prompt in prompts_of(name, [9, 40]):
        near_tie_follows(weights, config, prompt, model.generate(prompt, max_new_tokens=12))


def test_batch_of_prompts_equals_single_requests(model_folders):
    name = "tiny_b"
    model = model_for(name, model_folders[name], "float32")
    prompts = prompts_of(name, [1, 9, 40, 64, 100])
    together = model.generate(prompts, max_new_tokens=24)
    for p, out in zip(prompts, together):
        assert out == model.generate(p, max_new_tokens=24)


def test_temperature_with_seed_matches_plain(model_folders):
    name = "tiny_b"
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "float32")
    for i, prompt in enumerate(prompts_of(name, [9, 40])):
        want = plain.generate(weights, config, prompt, 24, temperature=0.7, seed=11 + i)
        got = model.generate(prompt, max_new_tokens=24, temperature=0.7, seed=11 + i)
        assert got == want
        again = model.generate(prompt, max_new_tokens=24, temperature=0.7, seed=11 + i)
        assert again == got                                   # the same seed, the same stream
    assert model.generate(prompt, max_new_tokens=24, temperature=0.7, seed=99) != got


def test_stop_token_is_emitted_and_ends(model_folders):
    name = "tiny_a"
    model = model_for(name, model_folders[name], "float32")
    prompt = prompts_of(name, [17])[0]
    free_run = model.generate(prompt, max_new_tokens=16)
    stop = free_run[5]
    first = free_run.index(stop)
    assert model.generate(prompt, max_new_tokens=16, stop_ids=[stop]) == free_run[:first + 1]


def test_page_pressure_changes_no_output(model_folders):
    """A pool so small (seven pages) that requests which were let in with room for their prompts
    outgrow it while they decode: the one admitted last is pushed out and recomputed."""
    name = "tiny_a"
    roomy = model_for(name, model_folders[name], "float32")
    tight = model_for(name, model_folders[name], "float32", max_tokens=112, max_requests=4)
    prompts = prompts_of(name, [30, 28, 33, 25], seed=8)
    want = [roomy.generate(p, max_new_tokens=40) for p in prompts]
    sched = tight.scheduler()
    ids = [sched.add_request(p, 40) for p in prompts]
    out = sched.run()
    assert sched.stats["pushed_out"] >= 1
    assert [out[i] for i in ids] == want
    tight.engine.cache.check()
    assert not tight.engine.cache.live


@pytest.mark.parametrize("name, seed", [("tiny_a", 1), ("tiny_b", 2), ("tiny_c", 3)])
def test_random_arrivals_under_random_settings(name, seed, model_folders):
    """Requests of random lengths that arrive while others run, under settings drawn at random: the page
    size, a pool of little more than the longest request (so that running requests are pushed out and
    recomputed), the number of live requests, the token budget, graphs and running ahead on or off.
    Greedy, float32: every output is the plain implementation's."""
    from fastllm_py_b200 import Model

    cfg = tiny.CONFIGS[name]["config"]
    weights, config = plain.load_folder(model_folders[name])
    rng = np.random.default_rng(seed)
    max_len = min(cfg.max_position_embeddings, 160)
    page = int(rng.choice([8, 16, 32]))
    requests = []
    for _ in range(int(rng.integers(8, 14))):
        new = int(rng.integers(1, 60))
        requests.append((rng.integers(0, cfg.vocab_size, size=int(rng.integers(1, max_len - new))).tolist(), new))
    pages_one = -(-max(len(p) + n for p, n in requests) // page)
    pool_pages = pages_one + int(rng.integers(0, max(2, pages_one)))
    budget = int(rng.choice([13, 32, 64]))
    model = Model.load(model_folders[name], dtype="float32", page_size=page, max_tokens=pool_pages * page,
                       max_requests=int(rng.integers(2, 7)), max_batched_tokens=max(budget, 16),
                       max_model_len=max_len, cuda_graph=bool(rng.random() < 0.6), check_cache=True)
    sched = model.scheduler(token_budget=budget, run_ahead=bool(rng.random() < 0.7))
    waiting, ids, outs, steps = list(enumerate(requests)), {}, {}, 0
    while waiting or sched.has_work():
        while waiting and (rng.random() < 0.4 or not sched.has_work()):
            i, (prompt, new) = waiting.pop(0)
            ids[sched.add_request(prompt, new)] = i
        for o in sched.step():
            if o.finished:
                outs[ids[o.request_id]] = list(sched.finished[o.request_id].output)
        steps += 1
        assert steps < 5000, "the scheduler makes no progress"
    model.engine.check_status()
    model.engine.cache.check()
    assert not model.engine.cache.live
    for i, (prompt, new) in enumerate(requests):
        assert outs[i] == plain.generate(weights, config, prompt, new), f"request {i} of {name}"


def near_tie_follows(weights, config, prompt, got):
    """bfloat16 greedy tokens follow the plain bfloat16-storage model; where the two part ways
    the plain model's two best logits must be nearly tied (within twice the storage noise)."""
    ids = list(prompt)
    for tok in got:
        row = plain.forward(weights, config, ids, store=plain.store_bf16)[-1]
        best = int(row.argmax())
        if tok != best:
            exact = plain.forward(weights, config, ids)[-1]
            spread = float((row - exact).abs().max())
            assert float(row[best] - row[tok]) <= 2 * spread + 1e-3
        ids.append(tok)


# The two schedules that the tiny configurations are specified with, through the scheduler on
# the GPU, against the plain implementation request by request.
SCHEDULES = {"tiny_a": dict(lengths=[5, 17, 33], budget=7, new=16),
             "tiny_b": dict(lengths=[1, 9, 40, 64, 100], budget=13, new=24)}


@pytest.mark.parametrize("name", list(SCHEDULES))
def test_prompts_together_in_portions_beside_decoding_float32(name, model_folders):
    """All prompts at once under a small token budget (portions of 13, or 7, beside the decode
    steps of the requests that are already through), greedy and at temperature 0.7 with a seed
    per request: the ids equal the plain implementation's, which generates one request at a time."""
    from fastllm_py_b200.sampling import SamplingParams

    sch = SCHEDULES[name]
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "float32")
    prompts = prompts_of(name, sch["lengths"], seed=21)
    for temperature in (0.0, 0.7):
        sched = model.scheduler(token_budget=sch["budget"])
        ids = [sched.add_request(p, sch["new"], SamplingParams(temperature=temperature, seed=100 + i))
               for i, p in enumerate(prompts)]
        out = sched.run()
        assert sched.stats["prefill_tokens"] == sum(sch["lengths"])
        assert sched.stats["steps"] > sum(sch["lengths"]) // sch["budget"]
        for i, (rid, p) in enumerate(zip(ids, prompts)):
            want = plain.generate(weights, config, p, sch["new"], temperature=temperature, seed=100 + i)
            assert out[rid] == want, f"{name} T={temperature} request {i}"
    model.engine.cache.check()
    assert not model.engine.cache.live


def test_prompts_together_in_portions_beside_decoding_bfloat16(model_folders):
    name = "tiny_b"
    sch = SCHEDULES[name]
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "bfloat16")
    prompts = prompts_of(name, sch["lengths"], seed=21)
    sched = model.scheduler(token_budget=sch["budget"])
    ids = [sched.add_request(p, sch["new"]) for p in prompts]
    out = sched.run()
    for rid, p in zip(ids, prompts):
        assert len(out[rid]) == sch["new"]
        near_tie_follows(weights, config, p, out[rid])


def test_page_pressure_changes_no_output_bfloat16(model_folders):
    """Push-out and recompute with everything on that serving has on: bfloat16 kernels, graph
    replay, decode steps launched ahead of the host.  Recomputing a pushed-out request runs its
    prompt and its produced tokens as one prompt, through other kernels than decoding them did,
    so a token may differ where the model's two best are nearly tied; anything else is equal."""
    name = "tiny_a"
    weights, config = plain.load_folder(model_folders[name])
    roomy = model_for(name, model_folders[name], "bfloat16")
    tight = model_for(name, model_folders[name], "bfloat16", max_tokens=112, max_requests=4)
    prompts = prompts_of(name, [30, 28, 33, 25], seed=8)
    want = [roomy.generate(p, max_new_tokens=40) for p in prompts]
    sched = tight.scheduler()
    assert sched.run_ahead and tight.engine.use_graph
    ids = [sched.add_request(p, 40) for p in prompts]
    out = sched.run()
    assert sched.stats["pushed_out"] >= 1
    for rid, p, w in zip(ids, prompts, want):
        assert len(out[rid]) == 40
        if out[rid] != w:
            near_tie_follows(weights, config, p, out[rid])
    tight.engine.cache.check()
    assert not tight.engine.cache.live


def test_command_line_generates_the_plain_tokens(model_folders):
    """bin/generate as a user runs it: MODEL PROMPT N DTYPE in fastllm-py's order
    (scripts/generate.py:16-19), the prompt given as token ids."""
    import subprocess
    import sys

    name = "tiny_b"
    weights, config = plain.load_folder(model_folders[name])
    prompt = prompts_of(name, [11], seed=33)[0]
    want = plain.generate(weights, config, prompt, 16)
    cmd = [sys.executable, str(tiny.ROOT / "bin" / "generate"), str(model_folders[name]), "-", "16", "float32",
           "--prompt-ids", ",".join(map(str, prompt)), "--page-size", "8", "--max-tokens", "256"]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert lines[0].startswith("[load ") and "3L hidden=96 heads=6/2 dtype=float32" in lines[0]
    assert [int(t) for t in lines[1].split(",")] == want
    assert lines[-1].startswith("[16 tokens in ") and lines[-1].endswith("tok/s]")
    # temperature with a seed, as the plain implementation draws
    want = plain.generate(weights, config, prompt, 12, temperature=0.7, seed=5)
    done = subprocess.run(cmd[:4] + ["12", "float32"] + cmd[6:] + ["--temperature", "0.7", "--seed", "5"],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert [int(t) for t in lines[1].split(",")] == want


def test_graphs_captured_before_a_scratch_buffer_grew_are_not_replayed(model_folders):
    """A small engine captures its decode step; then a larger engine of the same process makes
    the shared scratch buffers grow; the small engine's next steps must not replay graphs that
    point to the old buffers: it drops them, captures anew, and produces the same tokens as eager."""
    from fastllm_py_b200 import Model
    from fastllm_py_b200.native import scratch

    name = "tiny_c"
    prompts = prompts_of(name, [9, 40, 21], seed=2)
    page = tiny.CONFIGS[name]["page_size"]
    small = Model.load(model_folders[name], dtype="bfloat16", page_size=page, max_tokens=1024, max_requests=4,
                       max_batched_tokens=64, max_model_len=256)
    eager = small.generate(prompts, max_new_tokens=20, use_graph=False)
    assert small.generate(prompts, max_new_tokens=20) == eager
    assert len(small.engine._graphs) >= 1
    # ask for more than any engine so far has reserved (a buffer that nobody has needed yet is made first:
    # making one is no growth)
    dev = small.engine.device
    from fastllm_py_b200.native import attention, gemm_tc
    for buf in (gemm_tc.SCRATCH, attention.SCRATCH):
        scratch.get(dev, buf, 1)
    before = scratch.generation(dev)
    scratch.get(dev, gemm_tc.SCRATCH, scratch.size(dev, gemm_tc.SCRATCH) + 1)
    scratch.get(dev, attention.SCRATCH, scratch.size(dev, attention.SCRATCH) + 1)
    assert scratch.generation(dev) == before + 2
    assert small.generate(prompts, max_new_tokens=20) == eager
    assert small.engine.graphs_dropped >= 1 and len(small.engine._graphs) >= 1
    # small batch, large batch, small batch through one engine
    many = prompts_of(name, [5] * 4, seed=3)
    want_many = small.generate(many, max_new_tokens=8, use_graph=False)
    assert small.generate(prompts[:1], max_new_tokens=20) == eager[:1]
    assert small.generate(many, max_new_tokens=8) == want_many
    assert small.generate(prompts[:1], max_new_tokens=20) == eager[:1]


def test_graph_replay_equals_eager_bit_for_bit(model_folders):
    """The captured decode step against the same step run eagerly
    (the idea of fastllm_py/graph_decode.py:994-1032)."""
    from fastllm_py_b200 import StepEntry

    name = "tiny_b"
    rows = {}
    for use_graph in (False, True):
        model = model_for(name, model_folders[name], "bfloat16", cuda_graph=use_graph)
        eng = model.engine
        eng.use_graph = use_graph
        prompts = prompts_of(name, [7, 19, 3], seed=6)
        for i, p in enumerate(prompts):
            eng.begin(i)
            eng.step([StepEntry(i, p, [])])
        got = []
        for k in range(6):                                  # steps 0 (eager warm-up), 1 (capture), 2.. (replay)
            logits = eng.step([StepEntry(i, [(k * 7 + i) % 300], [0]) for i in range(3)])
            got.append(logits.to("cpu", copy=True))
        for i in range(3):
            eng.end(i)
        rows[use_graph] = got
    if True in rows and False in rows:
        for a, b in zip(rows[False], rows[True]):
            assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_of_prompt_portions(dtype, model_folders):
    """Equal portions of a long prompt are captured at their third occurrence and replayed;
    mixed steps run eagerly; bit for bit as without graphs either way."""
    from fastllm_py_b200 import StepEntry

    name = "tiny_c"
    cfg = tiny.CONFIGS[name]["config"]
    rng = np.random.default_rng(31)
    long_a = rng.integers(0, cfg.vocab_size, size=160).tolist()
    long_b = rng.integers(0, cfg.vocab_size, size=160).tolist()
    rows = {}
    for use_graph in (False, True):
        model = model_for(name, model_folders[name], dtype, cuda_graph=use_graph, max_tokens=2048)
        eng = model.engine
        eng.use_graph = use_graph
        got = []
        eng.begin("a")
        eng.begin("b")
        for k in range(5):                                  # five equal portions of 32 tokens: eager x2, capture, replay x2
            got.append(eng.step([StepEntry("a", long_a[32 * k:32 * k + 32], [31, 0])]).to("cpu", copy=True))
        if use_graph:
            assert len(eng._graphs) == 1
        for k in range(4):                                  # a portion of b beside one decoded token of a: always eager
            got.append(eng.step([StepEntry("b", long_b[24 * k:24 * k + 24], [23]),
                                 StepEntry("a", [(k * 11) % cfg.vocab_size], [0])]).to("cpu", copy=True))
        if use_graph:
            assert len(eng._graphs) == 1
        eng.end("a")
        eng.end("b")
        rows[use_graph] = got
    for a, b in zip(rows[False], rows[True]):
        assert torch.equal(a, b)


# ------------------------------------------------------------------- sampler

def test_sampler_matches_plain_sampler():
    from fastllm_py_b200.native import ops

    g = torch.Generator().manual_seed(0)
    vocab, rows = 1000, 64
    logits = (torch.randn(rows, vocab, generator=g) * 2.5)
    combos = [dict(), dict(top_k=7), dict(top_p=0.6), dict(min_p=0.15), dict(top_k=40, top_p=0.8, min_p=0.02),
              dict(top_k=1), dict(top_p=0.999)]
    rng = np.random.default_rng(1)
    for combo in combos:
        temp = 0.3 + 1.5 * rng.random(rows)
        uni = rng.random(rows)
        dev = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
        out = torch.zeros(rows, dtype=torch.int32, device=DEV)
        ops.sample(logits.to(DEV), out, dev(temp, torch.float32),
                   dev([combo.get("top_k", 0)] * rows, torch.int32),
                   dev([combo.get("top_p", 1.0)] * rows, torch.float32),
                   dev([combo.get("min_p", 0.0)] * rows, torch.float32), dev(uni, torch.float64))
        got = out.cpu().tolist()
        for r in range(rows):
            want = plain.sample(logits[r], float(np.float32(temp[r])), uniform=float(uni[r]), **combo)
            if got[r] != want:
                # only a draw that falls on the edge between two tokens may differ
                p = plain.probabilities(logits[r], float(np.float32(temp[r])), **combo)
                cdf = torch.cumsum(p, 0)
                assert p[got[r]] > 0, f"{combo}: token {got[r]} was filtered out"
                edge = cdf[min(got[r], want)]
                assert abs(float(edge) - uni[r]) < 1e-5, (combo, r, got[r], want)


def test_greedy_is_first_argmax_and_ignores_filters():
    from fastllm_py_b200.native import ops

    logits = torch.zeros(3, 500)
    logits[0, 77] = logits[0, 300] = 5.0                     # a tie: the first index wins
    logits[1, 499] = 1.0
    logits[2, 0] = 1.0
    out = torch.zeros(3, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), out)
    assert out.cpu().tolist() == [77, 499, 0]
    zero = torch.zeros(3, dtype=torch.float32, device=DEV)
    ops.sample(logits.to(DEV), out, zero, torch.full((3,), 5, dtype=torch.int32, device=DEV),
               torch.full((3,), 0.1, device=DEV), zero, torch.zeros(3, dtype=torch.float64, device=DEV))
    assert out.cpu().tolist() == [77, 499, 0]


def test_sampled_frequencies_follow_softmax():
    from fastllm_py_b200.native import ops

    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, 1.5]])
    n = 20000
    big = logits.repeat(n, 1).to(DEV)
    uni = torch.tensor(np.random.default_rng(3).random(n), dtype=torch.float64, device=DEV)
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.sample(big, out, torch.full((n,), 0.9, device=DEV), None, None, None, uni)
    freq = torch.bincount(out.cpu().long(), minlength=6).float() / n
    assert float((freq - torch.softmax(logits[0] / 0.9, 0)).abs().max()) < 0.02


def test_penalties_kernel():
    from fastllm_py_b200.native import ops

    g = torch.Generator().manual_seed(5)
    logits = torch.randn(2, 50, generator=g) * 3
    counts = [{3: 2, 7: 1, 49: 4}, {0: 1}]
    rep, freq, pres = [1.3, 1.0], [0.2, 0.0], [0.1, 0.5]
    items = [(r, t, c) for r, d in enumerate(counts) for t, c in d.items()]
    arr = torch.tensor(items, dtype=torch.int32).t().contiguous().to(DEV)
    dev = logits.to(DEV)
    f = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    ops.apply_penalties(dev, arr[0], arr[1], arr[2], f(rep), f(freq), f(pres))
    for r in range(2):
        want = plain.apply_penalties(logits[r], counts[r], rep[r], freq[r], pres[r])
        assert float((dev[r].cpu().double() - want).abs().max()) < 1e-5


def test_sampling_options_through_generate(model_folders):
    name = "tiny_a"
    weights, config = plain.load_folder(model_folders[name])
    model = model_for(name, model_folders[name], "float32")
    prompt = prompts_of(name, [12])[0]
    opts = dict(temperature=0.9, top_k=20, top_p=0.9, min_p=0.01, repetition_penalty=1.2,
                frequency_penalty=0.1, presence_penalty=0.1)
    got = model.generate(prompt, max_new_tokens=12, seed=3, **opts)
    # the plain loop with the same penalties and uniforms
    rng = np.random.default_rng(3)
    ids, counts, want = list(prompt), {}, []
    for _ in range(12):
        row = plain.forward(weights, config, ids)[-1]
        row = plain.apply_penalties(row, counts, 1.2, 0.1, 0.1)
        tok = plain.sample(row, 0.9, top_p=0.9, top_k=20, min_p=0.01, uniform=float(rng.random()))
        counts[tok] = counts.get(tok, 0) + 1
        want.append(tok)
        ids.append(tok)
    assert got == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_no_token(dtype, model_folders):
    """Decode steps launched before the tokens of the step before were read (the embedding
    takes them from the sampler's output on the device): same tokens as step by step, with
    requests of different lengths, one ended by a stop token in mid-flight (its row of the
    step under way is dropped), a late arrival, greedy and seeded sampling side by side."""
    from fastllm_py_b200.sampling import SamplingParams

    name = "tiny_b"
    model = model_for(name, model_folders[name], dtype)
    prompts = prompts_of(name, [7, 21, 40, 12, 3], seed=14)
    lengths = [30, 9, 22, 30, 17]
    params = [SamplingParams(), SamplingParams(temperature=0.8, seed=5), SamplingParams(),
              SamplingParams(temperature=1.1, top_k=20, seed=6), SamplingParams()]
    def run(run_ahead, stop=None):
        sched = model.scheduler(run_ahead=run_ahead)
        ids = [sched.add_request(p, n, s, stop_ids=[stop] if (i == 3 and stop is not None) else ())
               for i, (p, n, s) in enumerate(zip(prompts[:4], lengths, params))]
        steps = 0
        while sched.has_work():
            sched.step()
            steps += 1
            if steps == 24:                                # a late arrival breaks the steady state
                ids.append(sched.add_request(prompts[4], lengths[4], params[4]))
        return [sched.request(i).output for i in ids], dict(sched.stats)

    free = run(False)[0][3]                                # the sampled request, run to its length
    at = next(k for k in range(8, 22) if free.index(free[k]) == k)
    stop = free[at]                                        # it ends by this token, in the steady state

    want, plain_stats = run(False, stop)
    got, stats = run(True, stop)
    assert plain_stats["steps_ahead"] == 0
    assert stats["steps_ahead"] >= 10 and stats["rows_dropped"] >= 1
    assert got == want
    assert want[3] == free[:at + 1]
    model.engine.cache.check()
    assert not model.engine.cache.live
