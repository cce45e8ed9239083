"""Engine: the step function over a decoder and a cache manager.

`step(entries)` runs exactly the tokens it is given, as one batch, against what
earlier steps left in the cache, and returns the logits at the wanted places.
It neither samples nor decides what to run: the scheduler above it does, and so
does trace replay, through this same function.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from ..config.engine import EngineConfig
from ..native import scratch
from ..parts import BuildContext, Decoder, EngineLimits, Workspace
from .batch import StepBuffers, StepContext, build_views


@dataclass
class StepEntry:
    """A request's share of a step: its next tokens and the places (indices into
    `tokens`) whose logits are wanted."""
    request_id: object
    tokens: list
    want: list = field(default_factory=list)


class Engine:
    def __init__(self, decoder: Decoder, config: EngineConfig, max_model_len: int, num_pages: int):
        self.decoder = decoder
        self.config = config
        self.device = decoder.ctx.device
        self.dtype = decoder.ctx.dtype
        self.page_size = config.page_size
        self.max_model_len = max_model_len
        self.max_tokens = min(config.max_batched_tokens, 65535)
        bt_stride = -(-max_model_len // self.page_size)
        self.cache = CacheManager(decoder.cache_needs(), self.page_size, num_pages,
                                  config.max_requests, bt_stride,
                                  poison=config.cache_poison if config.check_cache else None)
        self.cache.allocate(self.device, self.dtype)
        self.workspace = Workspace(self.device, self.max_tokens)
        self.buffers = StepBuffers(self.device, self.max_tokens, config.max_requests,
                                   len(self.cache.groups), bt_stride)
        from ..native.gemm_tc import status_word
        self.status = status_word(self.device)
        # the error word's last copy on the host: refreshed after every step without waiting for it
        self.status_host = torch.zeros(1, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._status_pinned = self.status_host.is_pinned()
        self.no_rotation = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.vocab = decoder.vocab
        self.steps_run = 0
        # An int32 device tensor (the sampler's output) from which the embedding takes tokens that
        # the host has not read yet: a step may name such a token as -1 - row.  None: not offered.
        # Only an embedding part that says it understands such ids is ever given them.
        self.accepts_fed_tokens = decoder.takes_fed_tokens
        self._token_feed = None
        self.use_graph = bool(config.cuda_graph)
        self._graphs: dict = {}          # step shape -> (graph, logits view, kernels in it)
        self._graphs_generation = None   # the scratch generations the graphs in _graphs were captured under
        self._warmed: dict = {}          # step shape -> times seen before its capture
        self.max_graphs = 64
        self.graphs_dropped = 0          # graphs thrown away because a buffer they point to was replaced
        self._bt_rows: list = [None] * config.max_requests   # (request uid, table version) last written per row
        # every part sizes the scratch memory of its kernels now, so that nothing grows under a captured graph
        self.limits = EngineLimits(self.max_tokens, config.max_requests, max_model_len)
        decoder.reserve(self.limits, self.workspace)

    @property
    def token_feed(self):
        return self._token_feed

    @token_feed.setter
    def token_feed(self, tensor):
        if tensor is not None and not self.accepts_fed_tokens:
            raise RuntimeError("this model's embedding part does not take tokens from the device "
                               "(it does not declare takes_fed_tokens)")
        self._token_feed = tensor

    # -------------------------------------------------------------- requests
    def begin(self, request_id):
        """A request becomes live: it gets a state slot (pages come as it grows)."""
        return self.cache.admit(request_id)

    def end(self, request_id) -> None:
        """A request is finished or pushed out: its pages and slot go back."""
        self.cache.release(request_id)

    def is_live(self, request_id) -> bool:
        return request_id in self.cache.live

    def tokens_held(self, request_id) -> int:
        return self.cache.live[request_id].seq_len

    # ------------------------------------------------------------------ step
    def prepare(self, entries) -> StepContext:
        """Check the batch, take its pages, fill and upload the step's tables."""
        cache, buf = self.cache, self.buffers
        if not entries:
            raise ValueError("a step needs at least one entry")
        if len(entries) > self.config.max_requests:
            raise ValueError(f"{len(entries)} requests in one step; the engine allows "
                             f"{self.config.max_requests}")
        n_tokens = sum(len(e.tokens) for e in entries)
        if n_tokens > self.max_tokens:
            raise ValueError(f"{n_tokens} tokens in one step; the engine allows {self.max_tokens}")
        seen = set()
        need = 0
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if e.request_id not in cache.live:
                raise KeyError(f"request {e.request_id!r} is not live (call begin first)")
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            rc = cache.live[e.request_id]
            if rc.seq_len + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.request_id!r} would reach {rc.seq_len + len(e.tokens)} "
                                 f"tokens; the engine's longest sequence is {self.max_model_len}")
            lowest = min(e.tokens)
            if lowest < 0 and self.token_feed is not None:
                # -1 - r: the token the sampler chose in row r of its last launch, not read back yet
                lowest = -1 - lowest
                if lowest >= self.token_feed.numel():
                    raise ValueError(f"request {e.request_id!r}: fed-token row {lowest} is outside the "
                                     f"feed's {self.token_feed.numel()} rows")
                lowest = 0
            if lowest < 0 or max(e.tokens) >= self.vocab:
                raise ValueError(f"request {e.request_id!r}: a token id is outside the "
                                 f"vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} is outside its "
                                     f"{len(e.tokens)} tokens")
            need += cache.pages_missing(rc, len(e.tokens))
        for g in cache.groups:
            if g.pool.free_pages < need:
                raise OutOfPages(f"the step needs {need} more pages, {g.pool.free_pages} are free "
                                 f"of {g.pool.num_pages}")
        buf.wait_for_last_upload()
        tok = buf.host_view("token_ids")
        pos = buf.host_view("positions")
        treq = buf.host_view("tok_req")
        rows = buf.host_view("logit_rows")
        rstart = buf.host_view("req_start")
        rctx = buf.host_view("req_ctx")
        rqlen = buf.host_view("req_qlen")
        rslot = buf.host_view("req_slot")
        dec = buf.host_view("decode_tokens")
        n_dec = 0
        slot_views = [buf.host_view(f"slots{g}") for g in range(len(cache.groups))]
        bt_views = [buf.host_view(f"bt{g}").reshape(buf.max_requests, buf.bt_stride)
                    for g in range(len(cache.groups))]
        at, m = 0, 0
        bt_dirty = False
        q_lens, ctx_lens, slots_host = [], [], []
        for r, e in enumerate(entries):
            rc = cache.live[e.request_id]
            q = len(e.tokens)
            cache.extend(rc, q)
            tok[at:at + q] = e.tokens
            pos[at:at + q] = np.arange(rc.seq_len, rc.seq_len + q)
            treq[at:at + q] = r
            for w in e.want:
                rows[m] = at + int(w)
                m += 1
            for g in range(len(cache.groups)):
                cache.slot_mapping(g, rc, q, slot_views[g][at:at + q])
            if self._bt_rows[r] != (rc.uid, rc.version):   # the row on the device is stale
                for g in range(len(cache.groups)):
                    cache.block_table_row(g, rc, bt_views[g][r])
                self._bt_rows[r] = (rc.uid, rc.version)
                bt_dirty = True
            rstart[r], rctx[r], rqlen[r], rslot[r] = at, rc.seq_len, q, rc.slot
            if q == 1:
                dec[n_dec] = at
                n_dec += 1
            q_lens.append(q)
            ctx_lens.append(rc.seq_len)
            slots_host.append(rc.slot)
            at += q
        rstart[len(entries)] = at
        buf.upload(len(entries) if bt_dirty else 0)
        n = len(entries)
        step = StepContext(
            n_tokens=n_tokens, n_requests=n, n_wanted=m,
            token_ids=buf.dev_view("token_ids")[:n_tokens],
            positions=buf.dev_view("positions")[:n_tokens],
            tok_req=buf.dev_view("tok_req")[:n_tokens],
            logit_rows=buf.dev_view("logit_rows")[:m],
            req_start=buf.dev_view("req_start")[:n + 1],
            req_ctx=buf.dev_view("req_ctx")[:n],
            req_qlen=buf.dev_view("req_qlen")[:n],
            req_slot=buf.dev_view("req_slot")[:n],
            decode_tokens=buf.dev_view("decode_tokens")[:n_dec],
            status=self.status, workspace=self.workspace, no_rotation=self.no_rotation,
            q_lens=q_lens, ctx_lens=ctx_lens, slots_host=slots_host,
            max_q_len=max(q_lens), max_seq_len=max(c + q for c, q in zip(ctx_lens, q_lens)),
            n_decode_tokens=n_dec, token_feed=self.token_feed,
            rows_identity=(m == n_tokens and bool((rows[:m] == np.arange(m)).all())))
        step.for_graph = self.use_graph and step.max_q_len == 1 and self.decoder.graph_safe
        self.decoder.plan_step(step)
        step._views = build_views(cache, buf, n_tokens, n)
        return step

    def step(self, entries) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted places, vocab] on the
        device, ordered by entry and by `want`.  The tensor is a view of an
        engine buffer and is overwritten by the next step."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        step = self.prepare(entries)
        if self.use_graph and self.decoder.graph_safe:
            logits = self._with_graph(step)
        else:
            logits = self.decoder.forward(step)
        if self._status_pinned:
            self.status_host.copy_(self.status, non_blocking=True)     # read by `faulted` once the step is over
        for e in entries:
            self.cache.commit(self.cache.live[e.request_id], len(e.tokens))
        self.steps_run += 1
        return logits

    def _scratch_generation(self):
        return (scratch.generation(self.device), self.workspace.generation)

    def drop_stale_graphs(self) -> int:
        """Captured graphs hold the addresses of the buffers they were captured with.  When any
        such buffer has been replaced since (it grew), those graphs must never run again: all of
        them are dropped here, before the next replay or capture.  Returns how many went."""
        now = self._scratch_generation()
        dropped = 0
        if self._graphs_generation != now:
            dropped = len(self._graphs)
            self._graphs.clear()
            self._warmed.clear()
            self._graphs_generation = now
            self.graphs_dropped += dropped
        return dropped

    def _with_graph(self, step: StepContext) -> torch.Tensor:
        """A step replays a CUDA graph captured for its shape.  The first step of
        a shape runs eagerly (it sizes every buffer), a later one is captured,
        the ones after it are replayed: the step's inputs already sit in fixed
        device buffers, so a replay needs nothing but the upload that `prepare`
        did.  The shape is everything that the launches depend on: the numbers
        of tokens, requests, single-token requests and wanted rows, and what the
        mixers add (the attention part: how its decode kernel splits the keys).  A capture
        costs about as much as twenty steps save, so it is made where a shape
        is sure to come again: decode-only steps (hundreds alike; this is the
        captured decode step of fastllm_py/batched.py:230-275 with the LM head
        inside the graph) at their second occurrence, a lone request's prompt
        portion (equal portions of long prompts) at its third; other mixed
        steps run eagerly.  The least recently used graphs are dropped beyond
        `max_graphs`."""
        from ..native import ops

        feed = None if self.token_feed is None else self.token_feed.data_ptr()
        key = (step.n_tokens, step.n_requests, step.n_decode_tokens, step.n_wanted, step.rows_identity,
               self.decoder.graph_key(step), feed)
        self.drop_stale_graphs()
        entry = self._graphs.pop(key, None)
        if entry is not None:
            self._graphs[key] = entry                       # most recently used last
        if entry is None:
            if step.max_q_len == 1 and step.n_wanted == step.n_tokens:
                capture_at = 2
            elif step.n_requests == 1:
                capture_at = 3
            else:
                return self.decoder.forward(step)
            if len(self._warmed) > 4096:
                self._warmed.clear()
            seen = self._warmed[key] = self._warmed.get(key, 0) + 1
            if seen < capture_at:
                return self.decoder.forward(step)
            while len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            graph = torch.cuda.CUDAGraph()
            before = ops.counter.launches
            with torch.cuda.graph(graph):
                logits = self.decoder.forward(step)
            if self._scratch_generation() != self._graphs_generation:
                raise RuntimeError("a scratch buffer was replaced while a step was being captured")
            entry = self._graphs[key] = (graph, logits, ops.counter.launches - before)
            ops.counter.launches = before
        graph, logits, kernels = entry
        graph.replay()
        ops.counter.launches += kernels
        return logits

    def check_status(self) -> None:
        """Raise if a kernel reported a fault since the last check (synchronises)."""
        self._raise_for(int(self.status.item()))

    def faulted(self) -> None:
        """The same without waiting for the device: looks at the copy of the error word that
        every step sends to the host behind itself.  Call it after something else has waited
        for the step (the sampler's token read-back, say); then the copy is the step's own."""
        self._raise_for(int(self.status_host[0]))

    def _raise_for(self, code: int) -> None:
        if code != 0:
            self.status.zero_()
            self.status_host.zero_()
            raise RuntimeError(f"a kernel reported error code {code} (a token id outside the "
                               f"embedding table, or a wait that gave up); the tokens of this "
                               f"step and of any step after it are not to be trusted")
