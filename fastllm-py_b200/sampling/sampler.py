"""Sampling: options per request, random numbers on the host, the choice on the device.

The options and their meaning are fastllm-py's
(fastllm_py/graph_decode.py:73-133, fastllm_py/model.py:500-504):
temperature <= 0 is greedy (first index on ties) and ignores the filters;
otherwise penalties, temperature, top-k, min-p, top-p, then a categorical draw.
The reference draws with `numpy.random.default_rng(seed).choice(V, p=p)`, which
consumes one `rng.random()` per token and inverts the cumulative distribution;
here the host draws that same uniform number from the same generator and the
device kernel does the inversion, so that only the token id travels back.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..native import ops


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int | None = None

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0

    @property
    def penalized(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)


class SamplingState:
    """What sampling remembers of one request: its generator and what it produced."""

    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = np.random.default_rng(params.seed) if not params.greedy else None
        self.counts: dict = {}

    def next_uniform(self) -> float:
        return float(self.rng.random())

    def record(self, token: int) -> None:
        self.counts[token] = self.counts.get(token, 0) + 1


class Sampler:
    """Chooses one token per logits row on the device."""

    _FIELDS = (("uniform", np.float64), ("temperature", np.float32), ("top_p", np.float32),
               ("min_p", np.float32), ("repetition", np.float32), ("frequency", np.float32),
               ("presence", np.float32), ("top_k", np.int32))

    def __init__(self, device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self.offsets = {}
        off = 0
        for name, dt in self._FIELDS:
            self.offsets[name] = (off, dt)
            off += -(-(max_rows * np.dtype(dt).itemsize) // 16) * 16
        self.nbytes = off
        pin = torch.cuda.is_available()
        self.host = torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        # two host buffers: a launch may follow before the one before it was collected
        self.out_host = [torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._launches = 0
        self._params_uploaded = None                     # event: the staging areas may be rewritten after it
        # penalties: (row, token, count) triples of the tokens produced so far, staged like the rest
        self._pen_cap = 0
        self._pen_host = self._pen_dev = None
        self._grow_penalties(4096)

    def _grow_penalties(self, triples: int) -> None:
        """Room for `triples` (row, token, count) entries in pinned and in device memory; an upload
        still under way from the old staging area is waited for before it is let go."""
        if triples <= self._pen_cap:
            return
        if self._params_uploaded is not None:
            self._params_uploaded.synchronize()
        cap = max(triples, 2 * self._pen_cap)
        self._pen_host = torch.zeros((3, cap), dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self._pen_dev = torch.zeros((3, cap), dtype=torch.int32, device=self.device)
        self._pen_cap = cap

    def _host(self, name):
        off, dt = self.offsets[name]
        return self.host_np[off:off + self.max_rows * np.dtype(dt).itemsize].view(dt)

    def _dev(self, name, n):
        off, dt = self.offsets[name]
        tdt = {np.float64: torch.float64, np.float32: torch.float32, np.int32: torch.int32}[dt]
        return self.dev[off:off + self.max_rows * np.dtype(dt).itemsize].view(tdt)[:n]

    def sample(self, logits: torch.Tensor, states: list) -> list:
        """`logits` [m, vocab] float32 on the device (modified in place by
        penalties); `states` the m requests' SamplingState.  Returns m token ids
        and records them in the states."""
        return self.collect(self.launch(logits, states))

    def launch(self, logits: torch.Tensor, states: list):
        """Enqueues the choice of one token per row and its copy to the host; returns
        a handle for `collect`.  The chosen ids also stay in `self.out[:m]` on the
        device until the next launch.  Penalties use the tokens recorded so far, so
        a request with penalties must be collected before it is launched again."""
        m = logits.shape[0]
        if m != len(states):
            raise ValueError(f"{m} logits rows for {len(states)} requests")
        if m == 0:
            return (None, None, states)
        if m > self.max_rows:
            raise ValueError(f"{m} rows to sample; the sampler was made for {self.max_rows}")
        any_penalty = any(s.params.penalized and s.counts for s in states)
        any_random = any(not s.params.greedy for s in states)
        if any_penalty or any_random:
            if self._params_uploaded is not None:
                self._params_uploaded.synchronize()      # the last upload has left the staging area
            u, t = self._host("uniform"), self._host("temperature")
            tp, mp, tk = self._host("top_p"), self._host("min_p"), self._host("top_k")
            rep, fr, pr = self._host("repetition"), self._host("frequency"), self._host("presence")
            for i, s in enumerate(states):
                p = s.params
                t[i] = p.temperature if not p.greedy else 0.0
                u[i] = s.next_uniform() if not p.greedy else 0.0
                tp[i], mp[i], tk[i] = p.top_p, p.min_p, p.top_k
                rep[i], fr[i], pr[i] = p.repetition_penalty, p.frequency_penalty, p.presence_penalty
            self.dev.copy_(self.host, non_blocking=True)
            n_pen = 0
            if any_penalty:
                items = [(i, tok, cnt) for i, s in enumerate(states) if s.params.penalized
                         for tok, cnt in s.counts.items()]
                n_pen = len(items)
                self._grow_penalties(n_pen)
                self._pen_host.numpy()[:, :n_pen] = np.asarray(items, dtype=np.int32).T
                self._pen_dev[:, :n_pen].copy_(self._pen_host[:, :n_pen], non_blocking=True)
            if self._params_uploaded is None:
                self._params_uploaded = torch.cuda.Event()
            self._params_uploaded.record()
            if any_penalty:
                pen = self._pen_dev
                ops.apply_penalties(logits, pen[0, :n_pen], pen[1, :n_pen], pen[2, :n_pen],
                                    self._dev("repetition", m), self._dev("frequency", m),
                                    self._dev("presence", m))
        out = self.out[:m]
        if any_random:
            ops.sample(logits, out, self._dev("temperature", m), self._dev("top_k", m),
                       self._dev("top_p", m), self._dev("min_p", m), self._dev("uniform", m))
        else:
            ops.sample(logits, out)
        host = self.out_host[self._launches & 1]
        self._launches += 1
        host[:m].copy_(out, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return (host, done, states)

    def collect(self, handle) -> list:
        """Waits for a launch's token ids, records them in the states and returns them."""
        host, done, states = handle
        if host is None:
            return []
        done.synchronize()
        tokens = host[:len(states)].tolist()
        for s, tok in zip(states, tokens):
            s.record(tok)
        return tokens
