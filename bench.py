#!/usr/bin/env python
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]
                    [--workload decode|serve|67b]

The default run is the DeepSeek-LLM-7B sized model (30 layers, hidden 4096,
32 heads, head size 128, feed-forward 11008, vocabulary 102400) with random
bfloat16 weights: a batch of 8 requests, each with a 2048-token context already
in the cache, decoding one token per step.  A "step" is one decode step.  It
prints ONE line of JSON:

  value      decoded tokens per second, K steps timed on the device with CUDA
             events (the step function plus the sampling kernel, tokens given);
  e2e        the same through the public scheduler API: every step builds its
             batch on the host, copies it from pinned memory, runs, samples and
             reads the token ids back (the scheduler launches a decode step
             before it has read the tokens of the one before; K steps by wall
             clock, the median of three such passes);
  prefill    one 2048-token prompt in one step, 20 runs: tokens/s, ms (median;
             `ms_mean` beside it) and the fraction of the bfloat16 tensor-core
             peak that its FLOPs / time reach, timed after the decode runs (the
             GPU at its power cap, as a serving GPU is) and, as `*_before_decode`,
             before them;
  roofline   the decode step against HBM: bytes it has to read (every weight
             once, the cache of the live requests) / time / peak bandwidth;
  points     decode tokens/s at batch 1 and 64.

Weights (13.8 GB) and cache are far larger than the 126 MB L2, so no flush is
needed between steps.  Peaks come from MEASURED_PEAKS.json when the driver
wrote it, else from the fallback figures 6650 GB/s and 1590 TFLOP/s.

Two more workloads, each printing one line of its own:

  --workload serve   deepseek-coder-1.3b size (24 layers, hidden 2048, context 16384, linear
             rotary scaling 4): 128 requests with prompts of 64 to 8192 tokens and 32 to 512
             tokens to produce, Poisson arrivals (--rate a second), through the scheduler with a
             token budget of 2048 and a cache pool that holds a quarter of what all requests
             together would need; generated and prompt tokens a second, time to the first
             token, time between tokens, how often a request was pushed out;
  --workload tables  the headline model at other sizes: prompt steps of 128 to 8192 tokens, a 4096-token
             prompt in portions of 512, decode steps over a grid of batch sizes and context lengths;
  --workload 67b     deepseek-llm-67b size (95 layers, hidden 8192, 64 heads over 8 key/value
             heads; 135 GB of weights on the one GPU): a 2048-token prompt step and decode
             steps at batch 1, 8 and 16 with 4000-token contexts, with their roofline fractions.

fastllm-py's counterpart is scripts/bench_one.py:27-100 (128-token prefill, 64
decode steps, wall-clock per token); its lesson kept here is to time steady
steps only (docs/handoff-4090-ktransformers.md:45-48).
"""
import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL_7B = dict(num_layers=30, hidden_size=4096, num_heads=32, num_kv_heads=32, head_dim=128,
                intermediate_size=11008, vocab_size=102400, rope_theta=10000.0, rms_norm_eps=1e-6,
                max_position_embeddings=4096)
CONTEXT = 2048
PREFILL_TOKENS = 2048
PREFILL_REPEATS = 20
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs.  nvidia-smi takes
    a few tenths of a second to come up, so the sampler is started ahead of the region (`start`),
    the region is marked (`with sampler:`), and only the samples taken inside it count."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []                                    # (wall-clock second, fields)
        self.proc = None
        self.gpu = self._this_gpu()
        self.begin = self.end = None

    @staticmethod
    def _this_gpu() -> str:
        """The id nvidia-smi knows the timed device by: its UUID (under CUDA_VISIBLE_DEVICES cuda:0
        is usually not the machine's GPU 0, and the clocks of another user's GPU say nothing)."""
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:                                    # noqa: BLE001  (no device: nothing to sample)
            return "0"

    def start(self):
        if self.proc is not None:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __enter__(self):
        self.start()
        self.begin = time.time()
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7 and parts[1].isdigit():
                self.samples.append((time.time(), parts[1:]))

    def __exit__(self, *exc):
        self.end = time.time()
        if self.proc is not None:
            time.sleep(0.12)                                 # a last sample that was taken inside the region may still be on its way
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        # a sample is printed a moment after it was taken: allow for that at the region's end
        inside = [f for t, f in self.samples if self.begin <= t <= self.end + 0.06] if self.begin else []
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"], "gpu": self.gpu}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in inside)]
        return {"sm_mhz": int(statistics.median(int(s[0]) for s in inside)),
                "sm_max_mhz": int(inside[0][1]), "reasons": reasons,
                "samples": len(inside), "gpu": self.gpu}


def decode_bytes(cfg, batch, mean_context):
    """Bytes one decode step has to read: every weight it uses once (bf16), the
    embedding rows of its tokens, and the cached keys and values of its requests."""
    h, inter, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qkv = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    per_layer = h * qkv + cfg.num_heads * cfg.head_dim * h + 3 * h * inter + 2 * h
    weights = 2 * (cfg.num_layers * per_layer + h + v * h) + 2 * batch * h
    kv = batch * mean_context * cfg.num_layers * 2 * cfg.num_kv_heads * cfg.head_dim * 2
    return weights + kv


def prefill_flops(cfg, tokens):
    h, inter = cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    linear = 2 * tokens * (h * qkv + cfg.num_heads * cfg.head_dim * h + 3 * h * inter)
    attention = 2 * cfg.head_dim * cfg.num_heads * tokens * (tokens + 1)       # QK^T and PV, causal
    return cfg.num_layers * (linear + attention) + 2 * h * cfg.vocab_size


def fill_context(engine, rids, context, vocab, gen):
    """Put `context` random tokens of every request into the cache, in steps under the token budget."""
    import torch

    from fastllm_py_b200 import StepEntry

    for rid in rids:
        engine.begin(rid)
        at = 0
        while at < context:
            n = min(engine.max_tokens, context - at)
            toks = torch.randint(0, vocab, (n,), generator=gen).tolist()
            engine.step([StepEntry(rid, toks, [])])
            at += n


def time_decode(model, batch, steps, warmup, context, sample_clocks=False):
    """(tokens/s, ms per step, launches in the timed region, clocks) of device-timed decode steps."""
    import torch

    from fastllm_py_b200 import StepEntry
    from fastllm_py_b200.native import ops

    engine = model.engine
    vocab = engine.vocab
    gen = torch.Generator().manual_seed(batch)
    rids = [f"b{batch}_{i}" for i in range(batch)]
    sampler = ClockSampler().start() if sample_clocks else None      # up and sampling by the time the contexts are in
    fill_context(engine, rids, context, vocab, gen)
    tokens = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
    out = torch.zeros(batch, dtype=torch.int32, device=engine.device)

    def one(i):
        logits = engine.step([StepEntry(r, [tokens[i][j]], [0]) for j, r in enumerate(rids)])
        ops.sample(logits, out)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.__enter__()
    before = ops.counter.launches
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    launches = ops.counter.launches - before
    if sampler:
        sampler.__exit__()
    ms = start.elapsed_time(stop) / steps
    engine.check_status()
    for r in rids:
        engine.end(r)
    return batch * 1000.0 / ms, ms, launches, (sampler.summary() if sampler else None)


def time_e2e(model, batch, steps, warmup, context):
    """Decode tokens/s through the scheduler: host batch building, pinned upload, step, sampling, token read-back."""
    import torch

    sched = model.scheduler()
    gen = torch.Generator().manual_seed(1000 + batch)
    for i in range(batch):
        prompt = torch.randint(0, model.engine.vocab, (context,), generator=gen).tolist()
        sched.add_request(prompt, max_new_tokens=warmup + steps + 8)
    while any(r.remaining > 1 or not r.output for r in sched.requests.values()):
        sched.step()                                   # prompts in; every request now decodes
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    buf = model.engine.buffers
    bytes_before = buf.uploaded_bytes
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(sched.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (buf.uploaded_bytes - bytes_before) // steps
    for r in list(sched.running):
        model.engine.end(r.request_id)
    return produced / dt, h2d, 4 * batch + 4          # the token ids and the kernels' error word


def time_prefill(model, tokens, repeats, warmup):
    """(median, mean) milliseconds of one prompt step of `tokens` tokens over `repeats` runs."""
    import torch

    from fastllm_py_b200 import StepEntry

    engine = model.engine
    gen = torch.Generator().manual_seed(7)
    toks = torch.randint(0, engine.vocab, (tokens,), generator=gen).tolist()
    times = []
    for i in range(warmup + repeats):
        rid = f"p{i}"
        engine.begin(rid)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(rid, toks, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
        engine.end(rid)
    return statistics.median(times), statistics.fmean(times)


MODEL_1B3 = dict(num_layers=24, hidden_size=2048, num_heads=16, num_kv_heads=16, head_dim=128,
                 intermediate_size=5504, vocab_size=32256, rope_theta=100000.0, rms_norm_eps=1e-6,
                 max_position_embeddings=16384)
MODEL_67B = dict(num_layers=95, hidden_size=8192, num_heads=64, num_kv_heads=8, head_dim=128,
                 intermediate_size=22016, vocab_size=102400, rope_theta=10000.0, rms_norm_eps=1e-6,
                 max_position_embeddings=4096)


def percentiles(values):
    if not values:
        return None
    v = sorted(values)
    pick = lambda q: round(v[min(len(v) - 1, int(q * len(v)))], 2)
    return {"p50": pick(0.50), "p90": pick(0.90), "p99": pick(0.99)}


def serving_workload(seed, n_requests, rate_per_s, vocab):
    """[(arrival second, prompt ids, tokens to produce)]: prompt lengths uniform in [64, 8192], outputs
    uniform in [32, 512], Poisson arrivals, all from one seed."""
    import numpy as np

    rng = np.random.default_rng(seed)
    at, out = 0.0, []
    for _ in range(n_requests):
        at += float(rng.exponential(1.0 / rate_per_s))
        prompt = rng.integers(0, vocab, size=int(rng.integers(64, 8193))).tolist()
        out.append((at, prompt, int(rng.integers(32, 513))))
    return out


def run_serving(args):
    """Continuous batching of 128 requests at deepseek-coder-1.3b size through the scheduler: total
    tokens a second, time to the first token and between tokens, and how often a request was pushed
    out for want of pages (the pool holds a quarter of what all requests together would need)."""
    import torch

    from fastllm_py_b200 import LlamaConfig, Model
    from fastllm_py_b200.config.llama import LinearRopeScaling

    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=LinearRopeScaling(4.0),
                      tie_word_embeddings=False, **dict(MODEL_1B3, num_layers=args.layers or MODEL_1B3["num_layers"]))
    budget, pool, live = 2048, 256 * 1024, 64
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", page_size=16, max_tokens=pool, max_requests=live,
                              max_batched_tokens=budget, max_model_len=16384, cuda_graph=not args.no_graph)
    work = serving_workload(11, args.requests, args.rate, cfg.vocab_size)
    # warm-up: the same kinds of steps (portions, mixed, decode) on a few short requests, untimed
    warm = model.scheduler(token_budget=budget)
    for i in range(4):
        warm.add_request(work[i][1][:600 + 50 * i], max_new_tokens=24)
    warm.run()
    torch.cuda.synchronize()

    sched = model.scheduler(token_budget=budget)
    arrival, first, last, gaps, done_at = {}, {}, {}, [], {}
    nxt, produced = 0, 0
    sampler = ClockSampler()
    sampler.__enter__()
    t0 = time.perf_counter()
    while nxt < len(work) or sched.has_work():
        now = time.perf_counter() - t0
        while nxt < len(work) and work[nxt][0] <= now:
            rid = sched.add_request(work[nxt][1], max_new_tokens=work[nxt][2], arrival_time=work[nxt][0])
            arrival[rid] = work[nxt][0]
            nxt += 1
        if not sched.has_work():
            time.sleep(max(0.0, min(0.002, work[nxt][0] - now)))
            continue
        outs = sched.step()
        now = time.perf_counter() - t0
        for o in outs:
            produced += 1
            if o.request_id not in first:
                first[o.request_id] = now
            else:
                gaps.append((now - last[o.request_id]) * 1e3)
            last[o.request_id] = now
            if o.finished:
                done_at[o.request_id] = now
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    sampler.__exit__()
    model.engine.check_status()
    model.engine.cache.check()
    prompt_tokens = sum(len(w[1]) for w in work)
    line = {
        "metric": "continuous batching tok/s, deepseek-coder-1.3b size bf16, 128 requests, Poisson arrivals",
        "value": round(produced / elapsed, 1), "unit": "generated tokens/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "prompt_tokens_per_s": round(prompt_tokens / elapsed, 1), "seconds": round(elapsed, 2),
        "ttft_ms": percentiles([(first[r] - arrival[r]) * 1e3 for r in first]),
        "per_token_ms": percentiles(gaps),
        "latency_s": percentiles([done_at[r] - arrival[r] for r in done_at]),
        "pushed_out": sched.stats["pushed_out"], "steps": sched.stats["steps"],
        "steps_ahead": sched.stats["steps_ahead"], "finished": len(done_at),
        "config": {"model": "deepseek-coder-1.3b size, random weights", "layers": cfg.num_layers,
                   "requests": len(work), "arrivals_per_s": args.rate, "prompt_tokens": prompt_tokens,
                   "generated_tokens": produced, "token_budget": budget, "pool_tokens": pool,
                   "live_requests_most": live, "page_size": 16, "context_limit": 16384,
                   "cuda_graph": not args.no_graph},
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    return 0


def run_67b(args, warmup):
    """deepseek-llm-67b size on one GPU (135 GB of bfloat16 weights): a 2048-token prompt step and
    decode steps at batch 1, 8 and 16 with 4096-token contexts, device-timed, with their fractions of
    the tensor peak and of the HBM roofline."""
    import torch

    from fastllm_py_b200 import LlamaConfig, Model

    layers = args.layers or MODEL_67B["num_layers"]
    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=None, tie_word_embeddings=False,
                      **dict(MODEL_67B, num_layers=layers))
    pk = peaks()
    context, steps = 4000, max(8, min(args.steps, 32))      # (the model's limit is 4096 positions)
    pool = 16 * (context + warmup + steps + 64)
    t_load = time.time()
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", page_size=16, max_tokens=pool, max_requests=16,
                              max_batched_tokens=PREFILL_TOKENS, max_model_len=4096, cuda_graph=not args.no_graph)
    torch.cuda.synchronize()
    load_s = time.time() - t_load
    points = {}
    clocks = None
    for b in (8, 1, 16):
        v, ms, _, ck = time_decode(model, b, steps, warmup, context, sample_clocks=(b == 8))
        clocks = ck or clocks
        nbytes = decode_bytes(cfg, b, context + warmup + (steps + 1) / 2)
        points[f"decode_b{b}"] = {"value": round(v, 2), "ms_per_step": round(ms, 3),
                                  "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
    pms, _ = time_prefill(model, PREFILL_TOKENS, 5, 2)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    line = {
        "metric": "decode tok/s @ batch 8, 4000-token context, deepseek-llm-67b size bf16",
        "value": points["decode_b8"]["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": points["decode_b8"]["ms_per_step"], "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {"model": "deepseek-llm-67b size, random weights", "layers": layers,
                   "layers_of_config": MODEL_67B["num_layers"], "hidden": cfg.hidden_size, "heads": cfg.num_heads,
                   "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "seq_len": context, "page_size": 16, "prefill_tokens": PREFILL_TOKENS,
                   "cuda_graph": not args.no_graph, "peaks": pk["source"], "load_s": round(load_s, 1)},
        "points": points,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pms, 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                    "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def run_tables(args, warmup):
    """The other sizes of the headline model, one JSON line: a prompt step of 128 to 8192 tokens
    (whole, and a 4096-token prompt in portions of 512) with its fraction of the tensor peak, and
    decode steps over a grid of batch sizes and context lengths with their fractions of the HBM
    roofline.  Every figure that the design notes quote from these tables is in this line."""
    import torch

    from fastllm_py_b200 import LlamaConfig, Model, StepEntry

    layers = args.layers or MODEL_7B["num_layers"]
    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=None, tie_word_embeddings=False,
                      **dict(MODEL_7B, num_layers=layers, max_position_embeddings=16384))
    pk = peaks()
    grid = [(1, 512), (1, 4096), (1, 8192), (8, 512), (8, 4096), (8, 8192), (16, 8192), (32, 2048), (64, 512),
            (64, 2048), (128, 2048)]
    steps = max(8, min(args.steps, 32))
    pool = max(b * (c + warmup + steps + 64) for b, c in grid)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", page_size=16, max_tokens=pool, max_requests=128,
                              max_batched_tokens=8192, max_model_len=16384, cuda_graph=not args.no_graph)
    sampler = ClockSampler().start()
    sampler.__enter__()
    prompt = {}
    for t in (128, 256, 512, 1024, 2048, 4096, 8192):
        ms, mean = time_prefill(model, t, 10, 3)
        prompt[str(t)] = {"ms": round(ms, 3), "ms_mean": round(mean, 3),
                          "frac": round(prefill_flops(cfg, t) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    # a 4096-token prompt in eight portions of 512
    engine = model.engine
    toks = torch.randint(0, cfg.vocab_size, (4096,), generator=torch.Generator().manual_seed(3)).tolist()
    times = []
    for i in range(3 + 5):
        engine.begin("chunked")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for at in range(0, 4096, 512):
            engine.step([StepEntry("chunked", toks[at:at + 512], [511] if at + 512 == 4096 else [])])
        stop.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(stop))
        engine.end("chunked")
    chunked_ms = statistics.median(times)
    decode = {}
    for b, c in grid:
        v, ms, _, _ = time_decode(model, b, steps, warmup, c)
        nbytes = decode_bytes(cfg, b, c + warmup + (steps + 1) / 2)
        decode[f"{b}x{c}"] = {"ms_per_step": round(ms, 3), "value": round(v, 1),
                              "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
    sampler.__exit__()
    print(json.dumps({
        "metric": "prompt steps and decode steps at other sizes, DeepSeek-LLM-7B size bf16", "n_gpus": 1,
        "dtype": "bf16", "data": "synthetic", "impl": "ours", "steps": steps, "warmup": warmup,
        "config": {"model": "DeepSeek-LLM-7B size, random weights", "layers": layers,
                   "layers_of_config": MODEL_7B["num_layers"], "page_size": 16, "peaks": pk["source"],
                   "hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "cuda_graph": not args.no_graph},
        "prompt_step": prompt,
        "prompt_4096_in_portions_of_512": {"ms": round(chunked_ms, 3), "value": round(4096 * 1000.0 / chunked_ms, 1)},
        "decode": decode, "clocks": sampler.summary()}))
    return 0


def reference_cpu_path(ref_root, layers=1, context=256, decode_tokens=8):
    """fastllm-py's own NumPy model code (its CPU device, float32) timed at DeepSeek-LLM-7B layer
    sizes: `layers` of the 30 layers, one sequence (that path has no batch), a `context`-token
    prompt through Model.forward and `decode_tokens` greedy tokens one by one.  The package imports
    CuPy inside its functions; a stand-in module that maps the few names it uses onto NumPy lets
    the CPU path run where CuPy is absent (its GPU path cannot)."""
    import tempfile
    import types

    import numpy as np

    from fastllm_py_b200 import LlamaConfig
    from fastllm_py_b200.weights import write_model_folder

    if "cupy" not in sys.modules:
        cp = types.ModuleType("cupy")
        cp.ndarray = type("ndarray", (), {})
        cp.asnumpy = lambda x: np.asarray(x)
        cp.asarray = lambda x: np.asarray(x)
        cp.float32, cp.float16 = np.float32, np.float16
        sys.modules["cupy"] = cp
    sys.path.insert(0, str(ref_root))
    from fastllm_py import DeviceMap, Model

    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=None, tie_word_embeddings=False,
                      **dict(MODEL_7B, num_layers=layers))
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_model_folder(cfg, Path(tmp) / "model", seed=0, std=0.02, norm_std=0.02)
        model = Model.load(str(folder), DeviceMap({"cpu": 1}), dtype="float32")
        ids = np.random.default_rng(7).integers(0, cfg.vocab_size, size=context).astype(np.int64)
        t0 = time.perf_counter()
        logits, kvs = model.forward(ids)
        prefill_s = time.perf_counter() - t0
        nxt = int(np.asarray(logits[-1]).argmax())
        times = []
        for _ in range(decode_tokens):
            t0 = time.perf_counter()
            logits, kvs = model.forward(np.asarray([nxt]), kvs)
            nxt = int(np.asarray(logits[-1]).argmax())
            times.append(time.perf_counter() - t0)
    return {"device": "cpu (NumPy path of the reference, float32)", "layers": layers,
            "layers_of_config": MODEL_7B["num_layers"], "batch": 1, "context": context,
            "prefill_tok_s": round(context / prefill_s, 1),
            "decode_tok_s": round(1.0 / statistics.median(times), 2)}


def run_reference(args):
    """The reference arm: codemk8/fastllm-py as installed under baseline/_ref, through its own API.
    Its GPU path is CuPy (RawKernel, cuBLAS through cupy): it is tried whenever `import cupy` works;
    where it does not, the line says so (and, with --reference-cpu, carries the timing of the
    reference's CPU path at one layer of the same sizes, for scale: no ratio is meant by it)."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "fastllm_py").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "fastllm-py is not installed under baseline/_ref "
                          "(pip install --no-index --no-deps --target baseline/_ref of a copy of the reference)"}))
        return 0
    try:
        import cupy  # noqa: F401
        have_cupy = True
    except Exception as e:                                   # noqa: BLE001
        have_cupy, why = False, f"{type(e).__name__}: {e}"
    if not have_cupy:
        line = {"impl": "reference", "unavailable":
                "fastllm-py's GPU path needs CuPy (cupy-cuda12x), which cannot be imported here "
                f"({why}) and is not in the offline wheelhouse; the package itself installs with --no-deps"}
        if args.reference_cpu:
            try:
                line["cpu_path"] = reference_cpu_path(ref_root)
            except Exception as e:                           # noqa: BLE001
                line["cpu_path"] = {"failed": f"{type(e).__name__}: {e}"}
        print(json.dumps(line))
        return 0
    return run_reference_gpu(args, ref_root)


def run_reference_gpu(args, ref_root):
    """With CuPy at hand: the reference's own batched decoder (fastllm_py/batched.py:96-275) at the
    headline shape in float16 (it has no bfloat16), random weights written to a model folder."""
    import tempfile

    import numpy as np

    from fastllm_py_b200 import LlamaConfig
    from fastllm_py_b200.weights import write_model_folder

    sys.path.insert(0, str(ref_root))
    try:
        import cupy as cp
        from fastllm_py import DeviceMap, Model
        from fastllm_py.batched import BatchedDecoder

        layers = args.layers or MODEL_7B["num_layers"]
        cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=None, tie_word_embeddings=False,
                          **dict(MODEL_7B, num_layers=layers))
        warmup = max(3, args.warmup)
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_model_folder(cfg, Path(tmp) / "model", seed=0, std=0.02, norm_std=0.02)
            model = Model.load(str(folder), DeviceMap({"cuda:0": 1}), dtype="float16")
        rng = np.random.default_rng(8)
        prompts = [rng.integers(0, cfg.vocab_size, size=CONTEXT).astype(np.int64) for _ in range(args.batch)]
        dec = BatchedDecoder(model, args.batch, max_len=CONTEXT + warmup + args.steps + 8)
        dec.prime(prompts)
        tokens = np.zeros(args.batch, dtype=np.int64)
        for _ in range(warmup):
            dec.step(tokens)
        cp.cuda.Device().synchronize()
        start, stop = cp.cuda.Event(), cp.cuda.Event()
        start.record()
        for _ in range(args.steps):
            dec.step(tokens)
        stop.record()
        stop.synchronize()
        ms = cp.cuda.get_elapsed_time(start, stop) / args.steps
        print(json.dumps({"impl": "reference", "metric": "decode tok/s @ batch 8, 2048-token context, DeepSeek-LLM-7B",
                          "value": round(args.batch * 1000.0 / ms, 2), "unit": "tokens/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
                          "higher_is_better": True, "dtype": "fp16", "data": "synthetic",
                          "config": {"model": "DeepSeek-LLM-7B size, random weights", "global_batch": args.batch,
                                     "seq_len": CONTEXT, "layers": layers,
                                     "layers_of_config": MODEL_7B["num_layers"]}}))
    except Exception as e:                                   # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's GPU path failed: {type(e).__name__}: {e}"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers of the same sizes (the line names both numbers)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve", "67b", "tables"],
                    help="decode: the headline line (DeepSeek-LLM-7B size); serve: continuous batching at "
                         "deepseek-coder-1.3b size; 67b: prompt and decode steps at deepseek-llm-67b size")
    ap.add_argument("--requests", type=int, default=128, help="serve: how many requests")
    ap.add_argument("--rate", type=float, default=16.0, help="serve: mean arrivals a second")
    ap.add_argument("--reference-cpu", action="store_true",
                    help="--impl reference without CuPy: also time the reference's NumPy path (one layer, one sequence)")
    args = ap.parse_args()

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    if args.workload == "serve":
        return run_serving(args)
    if args.workload == "67b":
        return run_67b(args, warmup)
    if args.workload == "tables":
        return run_tables(args, warmup)
    args.layers = args.layers or MODEL_7B["num_layers"]

    import torch

    from fastllm_py_b200 import LlamaConfig, Model

    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=None, tie_word_embeddings=False,
                      **dict(MODEL_7B, num_layers=args.layers))
    pk = peaks()
    t_load = time.time()
    biggest = max(args.batch, 1 if args.no_points else 64)
    pool = biggest * (CONTEXT + warmup + args.steps + 64)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", page_size=16, max_tokens=pool,
                              max_requests=biggest, max_batched_tokens=PREFILL_TOKENS,
                              max_model_len=4096, cuda_graph=not args.no_graph)
    torch.cuda.synchronize()
    load_s = time.time() - t_load

    flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill_first = None
    if not args.no_points:
        # the prompt step once before the decode runs (the GPU has not yet reached its power cap) ...
        prefill_first = time_prefill(model, PREFILL_TOKENS, PREFILL_REPEATS, 3)
    value, ms, launches, clocks = time_decode(model, args.batch, args.steps, warmup, CONTEXT, True)
    mean_ctx = CONTEXT + warmup + (args.steps + 1) / 2
    nbytes = decode_bytes(cfg, args.batch, mean_ctx)
    achieved = nbytes / (ms * 1e-3) / 1e9
    # three passes of K steps each, the median reported: a pass of a quarter of a second now and then
    # catches a host hiccup of tens of milliseconds, which says nothing about the engine
    passes = sorted((time_e2e(model, args.batch, args.steps, warmup, CONTEXT) for _ in range(3)), key=lambda r: r[0])
    e2e, h2d, d2h = passes[1]
    line = {
        "metric": "decode tok/s @ batch 8, 2048-token context, DeepSeek-LLM-7B bf16",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "DeepSeek-LLM-7B size, random weights", "global_batch": args.batch,
                   "seq_len": CONTEXT, "parallelism": "single GPU", "layers": args.layers,
                   "layers_of_config": MODEL_7B["num_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "page_size": 16, "context_limit": 4096, "prefill_tokens": PREFILL_TOKENS,
                   "l2": "weights and cache exceed L2; no flush", "cuda_graph": not args.no_graph,
                   "peaks": pk["source"], "load_s": round(load_s, 1), "e2e_passes": 3},
        "e2e": {"value": round(e2e, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.no_points:
        # ... and again after them, where a serving GPU sits: this is the figure reported as `ms`
        pms, pmean = time_prefill(model, PREFILL_TOKENS, PREFILL_REPEATS, 3)
        frac = lambda t: round(flops / (t * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        line["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / pms, 1), "tokens": PREFILL_TOKENS,
                           "ms": round(pms, 3), "frac": frac(pms), "ms_mean": round(pmean, 3),
                           "repeats": PREFILL_REPEATS, "ms_before_decode": round(prefill_first[0], 3),
                           "ms_mean_before_decode": round(prefill_first[1], 3),
                           "frac_before_decode": frac(prefill_first[0]),
                           "frac_of_sustained": round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
        points = {}
        for b in (1, 64):
            v, _, _, _ = time_decode(model, b, max(8, args.steps // 2), warmup, CONTEXT)
            points[f"decode_b{b}"] = round(v, 2)
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
