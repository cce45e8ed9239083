"""Traces for replay tests: the same requests cut in different ways.

A trace is a list of steps in the format bin/trace_run reads:
    {"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}
Every builder wants the logits at every position of every request (so that the
first tokens of a sequence are covered too) unless `want_from` says otherwise;
results are keyed by (request id, absolute position).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def whole(requests: dict) -> list:
    """Each request alone and whole: one step each, all places wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "end": [rid],
                      "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}]})
    return steps


def tail_decode(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        toks = list(toks)
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}]})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "end": [rid] if i == len(toks) - 1 else [],
                          "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}]})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: dict, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 11)) -> list:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        toks = list(toks)
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            last = at + n == len(toks)
            steps.append({"step": len(steps), "end": [rid] if last else [],
                          "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}]})
            at += n
            k += 1
    return steps


def mixed(requests: dict, live: int = 4, seed: int = 0, prefill_sizes=(9, 2, 17, 5, 33),
          decode_tail: int = 12) -> list:
    """Up to `live` requests at a time: portions of some beside single tokens of
    others; a request that ends makes room for the next, so its pages are used
    again.  The last `decode_tail` tokens of each request come one per step."""
    rng = np.random.default_rng(seed)
    queue = [(rid, list(toks)) for rid, toks in requests.items()]
    active = {}                                   # rid -> [tokens, fed]
    steps = []
    k = 0
    while queue or active:
        while queue and len(active) < live:
            rid, toks = queue.pop(0)
            active[rid] = [toks, 0]
        entries, ended = [], []
        for rid in list(active):
            toks, fed = active[rid]
            if len(active) > 1 and rng.random() < 0.15:
                continue                          # a request may sit out a step
            left = len(toks) - fed
            if left <= decode_tail:
                n = 1
            else:
                n = min(prefill_sizes[k % len(prefill_sizes)], left - decode_tail)
                k += 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            active[rid][1] = fed + n
            if fed + n == len(toks):
                ended.append(rid)
                del active[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: list, granule: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to `granule`."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // granule) * granule for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def run_in_process(engine, steps: list) -> dict:
    """Drive an Engine directly; returns {(request, position): logits row (CPU float32)}."""
    from fastllm_py_b200 import StepEntry

    out, held = {}, {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not engine.is_live(e["id"]):
                engine.begin(e["id"])
                held[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = engine.step(entries).to("cpu", copy=True)
        row = 0
        for e in s["entries"]:
            for w in e["want"]:
                out[(e["id"], held[e["id"]] + w)] = logits[row]
                row += 1
            held[e["id"]] += len(e["tokens"])
        for rid in s["end"]:
            engine.end(rid)
            held.pop(rid, None)
    engine.check_status()
    engine.cache.check()
    return out


def run_program(model_folder, dtype: str, steps: list, out_dir, max_tokens: int, vocab: int,
                extra_args=()) -> dict:
    """Drive bin/trace_run as a subprocess, step by step, waiting for each `done`."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
                            env=dict(os.environ))
    out, held = {}, {}
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run said {line!r}"
            n_want = sum(len(e["want"]) for e in s["entries"])
            if n_want:
                data = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
                row = 0
                for e in s["entries"]:
                    base = held.get(e["id"], 0)
                    for w in e["want"]:
                        out[(e["id"], base + w)] = torch.from_numpy(data[row].copy())
                        row += 1
            for e in s["entries"]:
                held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
            for rid in s["end"]:
                held.pop(rid, None)
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return out
