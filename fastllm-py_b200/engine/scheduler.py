"""Scheduler: which requests run in the next step, and with how many tokens.

The successor of fastllm-py's `BatchedEngine` (fastllm_py/batched.py:321-403):
a FIFO queue, requests that join and leave between steps, a token per running
request per step, a request finished by a stop token (which is emitted) or by
`max_new_tokens`.  What is new:

  * a token budget per step; prompts are cut into portions under it and may
    span several steps, beside the decoded tokens of other requests (the
    reference prefills every prompt whole and alone, batched.py:372);
  * admission needs a free request slot, budget left, and free pages for the
    request's whole prompt and first token plus a page of growth for every
    request already running (with nothing running: just the pages of the
    first portion, the pool being all free);
  * bounds: a request whose prompt plus `max_new_tokens` exceeds the longest
    sequence, or the whole page pool, is refused when it is added.

When pages run out: running requests are served in the order they were
admitted; if one of them cannot get the pages for its next tokens, the request
admitted LAST is pushed out: its pages go back, it returns to the head of the
queue, and when it is admitted again its prompt and the tokens it already
produced are recomputed as one prompt (its output so far is kept; with a fixed
seed its sampling continues where it stopped, because the generator is kept
too).  While any request was pushed out in a step, no new request is admitted.

Running ahead.  In the steady state (every running request decoding, nobody
waiting, pages at hand) the next step does not need the host to know the tokens
just chosen: they sit in the sampler's output on the device, and the embedding
kernel can take them from there.  The scheduler then launches step n + 1 before
it reads the tokens of step n, so the host's share of a step (reading tokens,
finishing requests, building and uploading the next batch) runs while the GPU
works, instead of between two steps.  A request that ends by its length is
left out of step n + 1 beforehand; one that ends by a stop token is found out
one step late: its row of step n + 1 is computed for nothing and dropped.
`step()` returns the tokens of the step it collected, which is then the one
launched a call earlier.  Requests with penalties (which need the tokens on the
host), engines whose embedding part does not take tokens from the device, and
samplers without the device path run without it.

Faults.  Kernels whose bounded waits give up, and the embedding kernel when it
meets a token outside its table, set an error word on the device; every step
sends a copy of it to the host behind itself, and the scheduler looks at that
copy whenever it has read a step's tokens (every `status_every` steps), so that
generation stops with an error instead of going on with tokens that mean nothing.

Memory of the host.  A request is known to the scheduler while it waits or runs.
Once its last token has been handed out it moves to `finished`, which keeps the
most recent ones for inspection and forgets older ones, and its id may be used
again.
"""
from __future__ import annotations

from collections import OrderedDict, deque
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


@dataclass
class _InFlight:
    """A launched step whose chosen tokens the host has not read yet."""
    sampled: list                      # requests with a logits row, in row order
    handle: object                     # what the sampler's collect() takes; None: tokens already here
    tokens: list | None = None


class Scheduler:
    def __init__(self, engine, sampler, token_budget: int | None = None, run_ahead: bool = True):
        self.engine = engine
        self.sampler = sampler
        self.cache = engine.cache
        self.token_budget = token_budget or engine.max_tokens
        self.waiting: deque = deque()
        self.running: list = []                    # in order of admission
        self.requests: dict = {}                   # waiting or running
        self.finished: OrderedDict = OrderedDict() # the most recent `keep_finished` that ended
        self.keep_finished = 1024
        self.status_every = int(getattr(getattr(engine, "config", None), "status_every", 1) or 0)
        self._next_id = 0
        self.stats = {"steps": 0, "pushed_out": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "steps_ahead": 0, "rows_dropped": 0}
        self._flight: _InFlight | None = None
        # the device path for tokens: the engine's embedding reads the sampler's output
        feed = getattr(sampler, "out", None)
        self.run_ahead = bool(run_ahead and feed is not None and getattr(engine, "accepts_fed_tokens", False)
                              and hasattr(sampler, "launch") and hasattr(sampler, "collect"))
        if self.run_ahead:
            engine.token_feed = feed

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
        self.finished.pop(request_id, None)
        self.waiting.append(req)
        return request_id

    def request(self, request_id) -> Request:
        """A request that waits or runs, or one of the most recently finished."""
        req = self.requests.get(request_id)
        return req if req is not None else self.finished[request_id]

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._flight is not None)

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
            # Room for its whole prompt and its first token, and a page of growth for every request
            # already running: a request that is let in on the strength of its first portion alone is
            # the one pushed out again a few steps later, its portions computed for nothing.  With
            # nothing running the whole pool is free, and add_request has made sure that it fits.
            whole = -(-(req.remaining + 1) // self.cache.page_size)
            reserve = len(self.running)
            if self.running and any(g.pool.free_pages < whole + taken + reserve for g in self.cache.groups):
                break
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
        """Launch what can be launched, read one step's tokens; returns a StepOutput for
        each token read.  Without running ahead the step launched is the step read."""
        if self._flight is None:
            planned = self.plan()
            if not planned:
                if self.has_work():
                    raise RuntimeError("the scheduler has requests but can run none of them")
                return []
            self._flight = self._launch(planned)
        flight, self._flight = self._flight, None
        if self.run_ahead:
            ahead = self._plan_ahead(flight)
            if ahead:
                self._flight = self._launch_ahead(flight, ahead)
        return self._collect(flight)

    def _launch(self, planned) -> _InFlight:
        """A step whose tokens are all known to the host."""
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
        states = [r.sampling_state for r in sampled]
        if hasattr(self.sampler, "launch"):
            return _InFlight(sampled, self.sampler.launch(logits, states))
        return _InFlight(sampled, None, self.sampler.sample(logits, states))

    def _plan_ahead(self, flight: _InFlight) -> list:
        """The requests of the step after `flight`, if that step can be launched before
        `flight`'s tokens are read: [(request, its row in flight)], or [] to wait."""
        if self.waiting or not flight.sampled or len(flight.sampled) != len(self.running):
            return []
        row_of = {id(r): i for i, r in enumerate(flight.sampled)}
        ahead, taken = [], 0
        for req in self.running:                       # every running request must be one just sampled
            row = row_of.get(id(req))
            if row is None or req.sampling.penalized:
                return []
            produced = len(req.output) + 1             # with the token that is still on the device
            if produced >= req.max_new_tokens or len(req.prompt) + produced >= self.engine.max_model_len:
                continue                               # ends with that token: no next step for it
            rc = self.cache.live[req.request_id]
            if not self.cache.can_extend(rc, 1, spare=taken):
                return []                              # pages are short: decide with all tokens at hand
            taken += self.cache.pages_missing(rc, 1)
            ahead.append((req, row))
        return ahead

    def _launch_ahead(self, flight: _InFlight, ahead) -> _InFlight:
        """The next decode step of `ahead`'s requests; each one's token is named by its row
        in the sampler's last output (-1 - row), where the embedding kernel finds it."""
        entries = [StepEntry(req.request_id, [-1 - row], [0]) for req, row in ahead]
        logits = self.engine.step(entries)
        sampled = [req for req, _ in ahead]
        for req in sampled:
            req.computed += 1
        self.stats["decode_tokens"] += len(sampled)
        self.stats["steps_ahead"] += 1
        return _InFlight(sampled, self.sampler.launch(logits, [r.sampling_state for r in sampled]))

    def _collect(self, flight: _InFlight) -> list:
        tokens = flight.tokens if flight.handle is None else self.sampler.collect(flight.handle)
        outputs = []
        for req, tok in zip(flight.sampled, tokens):
            if req.finished:                           # ended by a stop token while this step was under way
                self.stats["rows_dropped"] += 1
                continue
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
                del self.requests[req.request_id]
                self.finished[req.request_id] = req
                while len(self.finished) > self.keep_finished:
                    self.finished.popitem(last=False)
            outputs.append(StepOutput(req.request_id, tok, bool(done)))
        self.stats["steps"] += 1
        if self.status_every and self.stats["steps"] % self.status_every == 0:
            check = getattr(self.engine, "faulted", None)
            if check is not None:
                check()                                # the tokens were waited for: the step's error word is here too
        return outputs

    def run(self, max_steps: int = 10_000_000, on_token=None) -> dict:
        """Step until nothing is left (or `max_steps`); returns request id -> produced tokens of
        every request that finished meanwhile and of those still waiting or running at the end."""
        result = {}
        steps = 0
        while self.has_work() and steps < max_steps:
            for out in self.step():
                if out.finished:
                    result[out.request_id] = self.finished[out.request_id].output
                if on_token is not None:
                    on_token(out)
            steps += 1
        for rid, req in self.requests.items():
            result[rid] = req.output
        return result
