"""Host-side rules of the engine that need no GPU: scratch buffers and captured graphs, the
cache's check mode, the error word in the scheduler, what the scheduler remembers, and what
parts declare."""
import numpy as np
import pytest
import torch

from fastllm_py_b200.cache import CacheManager, FixedState, PagedKV, PagedNeed
from fastllm_py_b200.config import EngineConfig
from fastllm_py_b200.engine import Engine
from fastllm_py_b200.engine.scheduler import Scheduler
from fastllm_py_b200.native import scratch
from fastllm_py_b200.parts import BuildContext, ResidualStream, Workspace

from test_cache_scheduler import ArgmaxSampler, FeedingEngine, LaunchingSampler, StandInEngine


# ------------------------------------------------ scratch buffers and captured graphs

def test_scratch_grows_once_and_says_so():
    dev = torch.device("cpu")
    g0 = scratch.generation(dev)
    a = scratch.get(dev, "test buffer", 100, at_least=256)
    assert a.numel() == 256 and scratch.generation(dev) == g0          # a first buffer replaces nothing
    assert scratch.get(dev, "test buffer", 200) is a                    # it is large enough: the same tensor
    b = scratch.get(dev, "test buffer", 1000)
    assert b.numel() >= 1000 and b is not a
    assert scratch.generation(dev) == g0 + 1                            # graphs captured with `a` are stale now
    scratch.reserve(dev, "test buffer", 500)
    assert scratch.generation(dev) == g0 + 1 and scratch.size(dev, "test buffer") == b.numel()


class _StubDecoder:
    """What an Engine asks of a decoder, without parts or kernels."""
    vocab, hidden, graph_safe, takes_fed_tokens = 32, 8, True, True

    def __init__(self):
        self.ctx = BuildContext(torch.device("cpu"), torch.float32, 4, 64)
        self.reserved = None

    def cache_needs(self):
        return {0: PagedKV(1, 16)}

    def reserve(self, limits, workspace):
        self.reserved = limits

    def plan_step(self, step):
        step.plans["stub"] = step.n_tokens

    def graph_key(self, step):
        return (step.plans["stub"],)


def _stub_engine(**options):
    config = EngineConfig(dtype="float32", page_size=4, max_requests=4, max_batched_tokens=16, device="cpu",
                          **options)
    return Engine(_StubDecoder(), config, max_model_len=64, num_pages=8)


def test_parts_reserve_their_scratch_when_the_engine_is_built():
    eng = _stub_engine()
    lim = eng.decoder.reserved
    assert (lim.max_tokens, lim.max_requests, lim.max_model_len) == (16, 4, 64)


def test_graphs_are_dropped_when_a_buffer_they_point_to_was_replaced():
    eng = _stub_engine()
    assert eng.drop_stale_graphs() == 0
    eng._graphs["a shape"] = ("graph", "logits", 3)
    eng._graphs["another"] = ("graph", "logits", 3)
    assert eng.drop_stale_graphs() == 0 and len(eng._graphs) == 2       # nothing grew: they stay
    # the split-K scratch of the device grows (another model, a larger step) ...
    scratch.get(eng.device, "split-K test", 10)
    scratch.get(eng.device, "split-K test", 10_000)
    assert eng.drop_stale_graphs() == 2 and not eng._graphs and eng.graphs_dropped == 2
    # ... and so does a workspace buffer of the engine itself
    eng._graphs["a shape"] = ("graph", "logits", 3)
    eng.workspace.rows("logits", 2, 32, torch.float32, initial=2)
    assert eng.drop_stale_graphs() == 0                                  # a first buffer replaces nothing
    eng.workspace.rows("logits", 9, 32, torch.float32, initial=2)
    assert eng.drop_stale_graphs() == 1 and not eng._graphs


def test_the_step_plan_comes_from_the_mixers():
    from fastllm_py_b200 import StepEntry

    eng = _stub_engine()
    eng.begin("r")
    step = eng.prepare([StepEntry("r", [1, 2, 3], [2])])
    assert step.plans == {"stub": 3} and not step.for_graph
    assert not hasattr(step, "decode_splits")                           # nothing of one mixer's kernel is in the batch form


def test_fed_tokens_are_a_capability_of_the_embedding():
    eng = _stub_engine()
    eng.token_feed = torch.zeros(4, dtype=torch.int32)
    eng.decoder.takes_fed_tokens = False
    eng2 = Engine(eng.decoder, eng.config, 64, 8)
    assert not eng2.accepts_fed_tokens
    with pytest.raises(RuntimeError, match="takes_fed_tokens"):
        eng2.token_feed = torch.zeros(4, dtype=torch.int32)
    # a scheduler over such an engine never launches ahead of the host
    plain_engine = StandInEngine(pages=16)
    assert not Scheduler(plain_engine, LaunchingSampler()).run_ahead
    assert Scheduler(FeedingEngine(pages=16), LaunchingSampler()).run_ahead


# ----------------------------------------------------------------- residual stream

class _Partial:
    def __init__(self, value):
        self.value = value

    def reduce_into(self, out):
        out.copy_(self.value)
        return out


def test_a_norm_that_does_not_take_partial_sums_gets_a_tensor():
    seen = []

    class PlainNorm:
        def apply(self, stream, out, rows=None):
            seen.append((type(stream.pending), rows))

    class PartialNorm(PlainNorm):
        takes_partial = True

    spill = torch.zeros(2, 3)
    value = torch.arange(6.0).reshape(2, 3)
    stream = ResidualStream(torch.zeros(2, 3), spill=lambda: spill)
    stream.pending = _Partial(value)
    stream.norm_into(PartialNorm(), None)
    assert seen[-1] == (_Partial, None)                                 # it adds the slabs itself
    stream.norm_into(PartialNorm(), None, rows=torch.tensor([1]))
    assert seen[-1][0] is torch.Tensor and torch.equal(stream.pending, value)   # gathered rows: summed up first
    stream.pending = _Partial(value + 1)
    stream.norm_into(PlainNorm(), None)
    assert seen[-1][0] is torch.Tensor and torch.equal(spill, value + 1)


# ------------------------------------------------------------------ cache: needs and check mode

class PagedVector(PagedNeed):
    """One vector per token (a need the package does not have)."""

    def __init__(self, dim, window=None):
        self.dim, self.window = dim, window

    def __eq__(self, other):
        return isinstance(other, PagedVector) and (self.dim, self.window) == (other.dim, other.window)

    def __hash__(self):
        return hash(("vec", self.dim, self.window))

    def page_shape(self, page_size):
        return (page_size, self.dim)


def test_a_need_states_its_page_shape_and_cost():
    assert PagedKV(2, 16).page_shape(8) == (2, 2, 8, 16)
    assert PagedKV(2, 16).bytes_per_token(8, 2) == 2 * 2 * 16 * 2
    assert PagedVector(24).bytes_per_token(8, 4) == 96
    needs = {0: PagedKV(2, 16), 1: PagedVector(24), 2: PagedVector(24), 3: FixedState((5,))}
    assert CacheManager.bytes_per_token(needs, 8, 2) == 128 + 48 + 48
    m = CacheManager(needs, 8, 6, 2, 4)
    m.allocate(torch.device("cpu"), torch.float32)
    assert [g.cache_ids for g in m.groups] == [[0], [1, 2]]
    assert tuple(m.groups[0].tensors[0].shape) == (6, 2, 2, 8, 16)
    assert tuple(m.groups[1].tensors[2].shape) == (6, 8, 24)


def test_check_mode_destroys_pages_that_go_back():
    needs = {0: PagedKV(1, 4), 1: PagedKV(1, 4, 6)}
    m = CacheManager(needs, 2, 8, 2, 16, poison=1.0e4)
    m.allocate(torch.device("cpu"), torch.float32)
    full, win = m.groups[0].tensors[0], m.groups[1].tensors[1]
    assert float(full.min()) == 1.0e4                                   # never-written places are poisoned too
    rc = m.admit("r")
    m.extend(rc, 12)
    for t in (full, win):
        t.zero_()                                                       # "the step wrote them"
    m.commit(rc, 12)
    # the window of 6 has passed tokens 0..5: logical pages 0..2 of the window group went back
    gone = [p for p in range(8) if p not in rc.pages[1]]
    assert len(gone) == 8 - 3 and m.pages_poisoned == 3
    assert all(float(win[p].min()) == 1.0e4 for p in gone if p < 6)
    assert all(float(win[p].abs().max()) == 0.0 for p in rc.pages[1] if p >= 0)
    assert float(full.abs().max()) == 0.0                               # the other group kept everything
    held = list(rc.pages[0])
    m.release("r")
    assert all(float(full[p].min()) == 1.0e4 for p in held)
    m.check()


# ---------------------------------------------------------------- scheduler: faults, memory

class FaultingEngine(StandInEngine):
    """Reports a kernel fault after its third step, the way Engine.faulted does."""

    def faulted(self):
        if len(self.steps) >= 3:
            raise RuntimeError("a kernel reported error code 101")


def test_generation_stops_when_a_kernel_reported_a_fault():
    s = Scheduler(FaultingEngine(pages=32), ArgmaxSampler())
    s.add_request([1, 2, 3], max_new_tokens=10)
    with pytest.raises(RuntimeError, match="error code 101"):
        s.run()
    assert s.stats["steps"] == 3                                        # no token was handed out after the fault


def test_the_error_word_reaches_the_host_copy():
    eng = _stub_engine()
    eng.faulted()                                                       # nothing recorded: no error
    eng.status_host[0] = 102
    with pytest.raises(RuntimeError, match="error code 102"):
        eng.faulted()
    eng.faulted()                                                       # raising cleared it


def test_finished_requests_are_forgotten_and_their_ids_free_again():
    eng = StandInEngine(pages=64, max_requests=4)
    s = Scheduler(eng, ArgmaxSampler())
    s.keep_finished = 3
    for round_ in range(5):
        ids = [s.add_request([1, 2, 3], max_new_tokens=2, request_id=f"r{k}") for k in range(3)]
        out = s.run()
        assert sorted(out) == sorted(ids) and all(len(v) == 2 for v in out.values())
        assert not s.requests and len(s.finished) <= 3
        assert s.request("r1").finish_reason == "length"
    with pytest.raises(KeyError):
        s.request("never seen")
