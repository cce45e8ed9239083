"""Scheduler: which requests run in the next step, and with how many tokens.

The successor of fastllm-py's `BatchedEngine` (fastllm_py/batched.py:321-403):
a FIFO queue, requests that join and leave between steps, a token per running
request per step, a request finished by a stop token (which is emitted) or by
`max_new_tokens`.  What is new:

  * a token budget per step; prompts are cut into portions under it and may
    span several steps, beside the decoded tokens of other requests (the
    reference prefills every prompt whole and alone, batched.py:372);
  * admission needs a free request slot, budget left, and pages for the first
    portion;
  * bounds: a request whose prompt plus `max_new_tokens` exceeds the longest
    sequence, or the whole page pool, is refused when it is added.

When pages run out: running requests are served in the order they were
admitted; if one of them cannot get the pages for its next tokens, the request
admitted LAST is pushed out: its pages go back, it returns to the head of the
queue, and when it is admitted again its prompt and the tokens it already
produced are recomputed as one prompt (its output so far is kept; with a fixed
seed its sampling continues where it stopped, because the generator is kept
too).  While any request was pushed out in a step, no new request is admitted.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..sampling import SamplingParams, SamplingState
from .engine import StepEntry


@dataclass
class Request:
    request_id: object
    prompt: list
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: frozenset = frozenset()
    arrival_time: float = 0.0
    # running state
    output: list = field(default_factory=list)
    computed: int = 0                   # tokens of prompt + output that are in the cache
    finished: bool = False
    finish_reason: str | None = None
    times_pushed_out: int = 0
    sampling_state: SamplingState | None = None

    @property
    def tokens(self):
        return self.prompt + self.output

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed


@dataclass
class StepOutput:
    request_id: object
    token: int
    finished: bool


class Scheduler:
    def __init__(self, engine, sampler, token_budget: int | None = None):
        self.engine = engine
        self.sampler = sampler
        self.cache = engine.cache
        self.token_budget = token_budget or engine.max_tokens
        self.waiting: deque = deque()
        self.running: list = []                    # in order of admission
        self.requests: dict = {}
        self._next_id = 0
        self.stats = {"steps": 0, "pushed_out": 0, "prefill_tokens": 0, "decode_tokens": 0}

    # ------------------------------------------------------------- requests
    def add_request(self, prompt, max_new_tokens: int = 32, sampling: SamplingParams | None = None,
                    stop_ids=(), request_id=None, arrival_time: float = 0.0):
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        total = len(prompt) + max_new_tokens
        if total > self.engine.max_model_len:
            raise ValueError(f"prompt ({len(prompt)}) + max_new_tokens ({max_new_tokens}) exceeds the "
                             f"longest sequence the engine holds ({self.engine.max_model_len})")
        pages = -(-total // self.cache.page_size)
        for g in self.cache.groups:
            if pages > g.pool.num_pages:
                raise ValueError(f"the request may need {pages} cache pages; the pool has "
                                 f"{g.pool.num_pages}, so it could never finish")
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        if request_id in self.requests:
            raise ValueError(f"request id {request_id!r} is already in use")
        req = Request(request_id, prompt, max_new_tokens, sampling or SamplingParams(),
                      frozenset(int(s) for s in (stop_ids or ())), arrival_time)
        req.sampling_state = SamplingState(req.sampling)
        self.requests[request_id] = req
        self.waiting.append(req)
        return request_id

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------- planning
    def _push_out(self, req: Request) -> None:
        self.engine.end(req.request_id)
        req.computed = 0
        req.times_pushed_out += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.stats["pushed_out"] += 1

    def plan(self):
        """[(request, tokens in this step)] for the next step.  Pushes requests
        out and admits new ones as a side effect."""
        pushed = False
        while True:
            budget = self.token_budget
            planned = []
            taken = 0                                   # pages this step's earlier entries will take
            starved = None
            for req in self.running:
                if budget <= 0:
                    break
                n = min(req.remaining, budget)
                rc = self.cache.live[req.request_id]
                if not self.cache.can_extend(rc, n, spare=taken):
                    starved = req
                    break
                taken += self.cache.pages_missing(rc, n)
                planned.append((req, n))
                budget -= n
            if starved is None:
                break
            victim = self.running[-1]
            self._push_out(victim)
            pushed = True
            if not self.running:
                # the victim was the only running request: it is re-admitted below
                # with the whole pool free, and add_request guaranteed that it fits
                planned, budget, taken = [], self.token_budget, 0
                pushed = False
                break
        while (self.waiting and not pushed and budget > 0
               and self.cache.slots.free_slots > 0):
            req = self.waiting[0]
            n = min(req.remaining, budget)
            pages = -(-n // self.cache.page_size)
            if any(g.pool.free_pages < pages + taken for g in self.cache.groups):
                break
            self.waiting.popleft()
            self.engine.begin(req.request_id)
            self.running.append(req)
            taken += pages
            planned.append((req, n))
            budget -= n
        return planned

    # ----------------------------------------------------------------- step
    def step(self) -> list:
        """Run one step of the engine; returns a StepOutput for each token produced."""
        planned = self.plan()
        if not planned:
            if self.has_work():
                raise RuntimeError("the scheduler has requests but can run none of them")
            return []
        entries, sampled = [], []
        for req, n in planned:
            lp = len(req.prompt)
            if req.computed >= lp:
                toks = req.output[req.computed - lp:req.computed - lp + n]
            elif req.computed + n <= lp:
                toks = req.prompt[req.computed:req.computed + n]
            else:
                toks = req.tokens[req.computed:req.computed + n]
            last = req.computed + n == lp + len(req.output)
            entries.append(StepEntry(req.request_id, toks, [n - 1] if last else []))
            if last:
                sampled.append(req)
            if n == 1 and req.output and req.computed + 1 == len(req.prompt) + len(req.output):
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += n
        logits = self.engine.step(entries)
        for req, n in planned:
            req.computed += n
        tokens = self.sampler.sample(logits, [r.sampling_state for r in sampled])
        outputs = []
        for req, tok in zip(sampled, tokens):
            req.output.append(tok)
            done = None
            if tok in req.stop_ids:
                done = "stop"
            elif len(req.output) >= req.max_new_tokens:
                done = "length"
            elif len(req.prompt) + len(req.output) >= self.engine.max_model_len:
                done = "max_model_len"
            if done:
                req.finished, req.finish_reason = True, done
                self.engine.end(req.request_id)
                self.running.remove(req)
            outputs.append(StepOutput(req.request_id, tok, bool(done)))
        self.stats["steps"] += 1
        return outputs

    def run(self, max_steps: int = 10_000_000, on_token=None) -> dict:
        """Step until nothing is left; returns request id -> produced tokens."""
        steps = 0
        while self.has_work() and steps < max_steps:
            for out in self.step():
                if on_token is not None:
                    on_token(out)
            steps += 1
        return {rid: req.output for rid, req in self.requests.items()}
