"""The cache manager's books and the scheduler's decisions (no GPU).

The scheduler runs here against the real CacheManager and a stand-in engine
whose "model" emits a fixed function of the request's token count, so that its
decisions (admission, portions under the budget, finishing, pushing out when
pages run out) can be checked exactly.
"""
import random

import numpy as np
import pytest
import torch

from fastllm_py_b200.cache import CacheManager, FixedState, OutOfPages, PagedKV, PagePool
from fastllm_py_b200.engine.scheduler import Scheduler
from fastllm_py_b200.sampling import SamplingParams


# ------------------------------------------------------------------ page pool

def test_pool_refuses_without_side_effects():
    pool = PagePool(4)
    a = pool.take(3)
    with pytest.raises(OutOfPages):
        pool.take(2)
    assert pool.free_pages == 1
    pool.give_back(a)
    with pytest.raises(RuntimeError, match="twice"):
        pool.give_back([a[0]])
    pool.check()


def manager(pages=16, page_size=4, window=None, max_requests=4, max_pages=64):
    needs = {0: PagedKV(2, 16), 1: PagedKV(2, 16)}
    if window:
        needs[2] = PagedKV(2, 16, window)
    needs[3] = FixedState((5,))
    return CacheManager(needs, page_size, pages, max_requests, max_pages)


def test_groups_by_need_and_state_slots():
    m = manager(window=6)
    assert [g.cache_ids for g in m.groups] == [[0, 1], [2]]
    assert m.state_needs == {3: FixedState((5,))}
    a, b = m.admit("a"), m.admit("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(RuntimeError):
        m.admit("a")
    m.release("a")
    assert m.admit("c").slot == a.slot                     # a freed slot is used again
    m.check()


def test_extend_commit_tables():
    m = manager(pages=8, page_size=4)
    rc = m.admit("r")
    m.extend(rc, 6)
    assert len(rc.pages[0]) == 2 and m.groups[0].pool.free_pages == 6
    slots = np.zeros(6, dtype=np.int32)
    m.slot_mapping(0, rc, 6, slots)
    p0, p1 = rc.pages[0]
    assert slots.tolist() == [p0 * 4, p0 * 4 + 1, p0 * 4 + 2, p0 * 4 + 3, p1 * 4, p1 * 4 + 1]
    m.commit(rc, 6)
    m.extend(rc, 1)                                        # token 7 fits the second page
    assert len(rc.pages[0]) == 2
    m.commit(rc, 1)
    m.extend(rc, 2)                                        # token 9 needs a third
    assert len(rc.pages[0]) == 3
    row = np.zeros(m.max_pages_per_request, dtype=np.int32)
    m.block_table_row(0, rc, row)
    assert row.tolist() == rc.pages[0] + [-1] * (m.max_pages_per_request - 3)
    with pytest.raises(RuntimeError):
        m.commit(rc, 9)                                    # more tokens than pages were taken for
    m.check()


def test_out_of_pages_takes_nothing():
    m = manager(pages=3, page_size=4)
    a, b = m.admit("a"), m.admit("b")
    m.extend(a, 8)
    assert not m.can_extend(b, 8) and m.can_extend(b, 4)
    with pytest.raises(OutOfPages):
        m.extend(b, 8)
    assert b.pages[0] == [] and m.groups[0].pool.free_pages == 1
    m.release("a")
    m.extend(b, 8)
    m.check()


def test_request_length_limit():
    m = manager(pages=64, page_size=4, max_pages=3)
    rc = m.admit("r")
    assert not m.can_extend(rc, 13)
    with pytest.raises(OutOfPages, match="most a request may hold"):
        m.extend(rc, 13)


def test_window_gives_pages_back():
    m = manager(pages=8, page_size=4, window=6)
    full, win = m.groups
    rc = m.admit("r")
    for _ in range(5):                                     # 20 tokens, 4 at a time
        m.extend(rc, 4)
        m.commit(rc, 4)
    # next query at 20 sees keys 15..20: pages 0..2 (positions 0..11) are dead
    assert rc.pages[1][:3] == [-1, -1, -1] and all(p >= 0 for p in rc.pages[1][3:])
    assert win.pool.held_pages == 2 and full.pool.held_pages == 5
    m.check()
    m.release("r")
    assert win.pool.free_pages == 8 and full.pool.free_pages == 8


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager(pages=24, page_size=4, window=9, max_requests=5)
    live = {}
    for step in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{step}"
            live[rid] = m.admit(rid)
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 11])
            if m.can_extend(live[rid], n):
                m.extend(live[rid], n)
                m.commit(live[rid], n)
            else:
                with pytest.raises(OutOfPages):
                    m.extend(live[rid], n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.pool.free_pages == 24 for g in m.groups) and m.slots.free_slots == 5


# ------------------------------------------------------------------ scheduler

class StandInEngine:
    """Real cache manager, no model: the logits of a wanted row make argmax equal
    (tokens the request holds after the step) mod vocab."""
    vocab = 50

    def __init__(self, pages, page_size=4, max_requests=4, max_model_len=64, max_tokens=16):
        self.cache = CacheManager({0: PagedKV(1, 16)}, page_size, pages, max_requests,
                                  -(-max_model_len // page_size))
        self.max_model_len = max_model_len
        self.max_tokens = max_tokens
        self.steps = []

    def begin(self, rid):
        return self.cache.admit(rid)

    def end(self, rid):
        self.cache.release(rid)

    def step(self, entries):
        rows = []
        self.steps.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        assert sum(len(e.tokens) for e in entries) <= self.max_tokens
        for e in entries:
            rc = self.cache.live[e.request_id]
            self.cache.extend(rc, len(e.tokens))
            self.cache.commit(rc, len(e.tokens))
            for _ in e.want:
                row = torch.zeros(self.vocab)
                row[rc.seq_len % self.vocab] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, self.vocab)


class ArgmaxSampler:
    def sample(self, logits, states):
        toks = logits.argmax(-1).tolist()
        for s, t in zip(states, toks):
            s.record(t)
        return toks


def test_portions_under_the_budget_and_first_token():
    eng = StandInEngine(pages=32, max_tokens=8)
    s = Scheduler(eng, ArgmaxSampler(), token_budget=8)
    rid = s.add_request(list(range(19)), max_new_tokens=3)
    out = s.run()
    # 19 prompt tokens under a budget of 8: portions 8, 8, 3; only the last wants logits
    assert eng.steps[:3] == [[(rid, 8, [])], [(rid, 8, [])], [(rid, 3, [2])]]
    assert eng.steps[3:] == [[(rid, 1, [0])], [(rid, 1, [0])]]
    assert out[rid] == [19, 20, 21]
    assert not eng.cache.live and eng.cache.groups[0].pool.free_pages == 32


def test_decodes_run_beside_a_prompt_portion():
    eng = StandInEngine(pages=32, max_tokens=8)
    s = Scheduler(eng, ArgmaxSampler(), token_budget=8)
    a = s.add_request([1, 2, 3], max_new_tokens=4)
    s.step()                                              # a: prompt whole, first token
    b = s.add_request(list(range(12)), max_new_tokens=2)
    s.step()
    # a decodes one token, b gets the rest of the budget
    assert eng.steps[1] == [(a, 1, [0]), (b, 7, [])]
    s.step()
    assert eng.steps[2] == [(a, 1, [0]), (b, 5, [4])]
    s.run()
    assert len(s.request(a).output) == 4 and len(s.request(b).output) == 2


def test_stop_token_is_emitted_and_ends_the_request():
    eng = StandInEngine(pages=32)
    s = Scheduler(eng, ArgmaxSampler())
    rid = s.add_request([7, 7, 7], max_new_tokens=10, stop_ids=[5])
    out = s.run()
    assert out[rid] == [3, 4, 5] and s.request(rid).finish_reason == "stop"


def test_requests_that_can_never_fit_are_refused():
    eng = StandInEngine(pages=4, page_size=4, max_model_len=64)
    s = Scheduler(eng, ArgmaxSampler())
    with pytest.raises(ValueError, match="never finish"):
        s.add_request(list(range(10)), max_new_tokens=8)      # 18 tokens > 16 in the pool
    with pytest.raises(ValueError, match="longest sequence"):
        s.add_request(list(range(60)), max_new_tokens=8)
    with pytest.raises(ValueError):
        s.add_request([], max_new_tokens=1)


def test_admission_waits_for_slots_and_pages():
    eng = StandInEngine(pages=6, page_size=4, max_requests=2)
    s = Scheduler(eng, ArgmaxSampler())
    ids = [s.add_request([1] * 6, max_new_tokens=2) for _ in range(3)]
    s.step()
    assert [r.request_id for r in s.running] == ids[:2] and len(s.waiting) == 1   # two slots only
    s.run()
    assert all(len(s.request(i).output) == 2 for i in ids)
    assert eng.cache.groups[0].pool.free_pages == 6


def test_admission_wants_room_for_the_whole_prompt():
    """A long prompt is let in when the free pages hold all of it, its first token and a page of
    growth for each running request, not on the strength of its first portion alone (it would be
    the next one pushed out, its portions computed for nothing); with nothing running it is let
    in whatever the budget cuts it into."""
    eng = StandInEngine(pages=10, page_size=4, max_requests=4, max_model_len=64, max_tokens=8)
    s = Scheduler(eng, ArgmaxSampler(), token_budget=8)
    a = s.add_request([1] * 10, max_new_tokens=9)            # 3 pages now, up to 5
    s.step()
    s.step()                                                 # a's prompt is in: it decodes
    b = s.add_request([2] * 29, max_new_tokens=2)            # 8 pages for prompt + first token
    s.step()
    assert [r.request_id for r in s.running] == [a], "7 free pages hold b's first portion, not b"
    out = s.run()
    assert len(out[a]) == 9 and len(out[b]) == 2 and s.stats["pushed_out"] == 0
    assert eng.cache.groups[0].pool.free_pages == 10
    lone = Scheduler(StandInEngine(pages=8, page_size=4, max_tokens=8), ArgmaxSampler(), token_budget=8)
    c = lone.add_request([3] * 29, max_new_tokens=2)
    lone.step()
    assert [r.request_id for r in lone.running] == [c]


def test_pages_run_out_last_admitted_is_pushed_out_and_recomputed():
    # 6 pages of 4 tokens; two requests of 7 prompt tokens (2 pages each) that decode
    # 8 more (up to 15 tokens = 4 pages each): together they need 8 pages, so one must go.
    eng = StandInEngine(pages=6, page_size=4, max_requests=4)
    s = Scheduler(eng, ArgmaxSampler())
    a = s.add_request([1] * 7, max_new_tokens=8)
    b = s.add_request([2] * 7, max_new_tokens=8)
    out = s.run()
    assert s.stats["pushed_out"] >= 1
    assert s.request(b).times_pushed_out >= 1 and s.request(a).times_pushed_out == 0
    # outputs are what an undisturbed run gives: token = tokens held after the step
    assert out[a] == list(range(7, 15)) and out[b] == list(range(7, 15))
    # b's comeback recomputed prompt + produced tokens as one prompt
    regrown = [st for st in eng.steps if any(r == b and n > 7 for r, n, _ in st)]
    assert regrown, "the pushed-out request did not come back with its produced tokens"
    assert not eng.cache.live and eng.cache.groups[0].pool.free_pages == 6


def test_no_admission_while_a_request_was_pushed_out():
    eng = StandInEngine(pages=6, page_size=4, max_requests=4)
    s = Scheduler(eng, ArgmaxSampler())
    s.add_request([1] * 7, max_new_tokens=8)
    s.add_request([2] * 7, max_new_tokens=8)
    c = s.add_request([3] * 3, max_new_tokens=1)
    seen_push = False
    while s.has_work():
        before = s.stats["pushed_out"]
        running_before = {r.request_id for r in s.running}
        s.step()
        if s.stats["pushed_out"] > before:
            seen_push = True
            admitted = {r.request_id for r in s.running} - running_before
            assert not admitted, "a request was admitted in a step that pushed one out"
    assert seen_push and len(s.request(c).output) == 1


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_with_clean_books(seed):
    rng = random.Random(seed)
    eng = StandInEngine(pages=10, page_size=4, max_requests=3, max_model_len=40, max_tokens=12)
    s = Scheduler(eng, ArgmaxSampler(), token_budget=12)
    want = {}
    for _ in range(12):
        n, m = rng.randint(1, 20), rng.randint(1, 12)
        rid = s.add_request([0] * n, max_new_tokens=m)
        want[rid] = [(n + i) % 50 for i in range(m)]
    out = s.run(max_steps=2000)
    assert out == want
    assert not s.has_work() and not eng.cache.live
    assert eng.cache.groups[0].pool.free_pages == 10 and eng.cache.slots.free_slots == 3


def test_sampling_params():
    assert SamplingParams().greedy and not SamplingParams(temperature=0.5).greedy
    assert SamplingParams(presence_penalty=0.1).penalized and not SamplingParams().penalized


# ------------------------------------------------- running one decode step ahead

class FeedingEngine(StandInEngine):
    """A stand-in for the device path: a token named -1 - row is taken from the sampler's last
    output, as the embedding kernel does; the logits depend on the tokens a request was fed,
    so a wrongly fed token changes every later one."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.token_feed = None
        self.accepts_fed_tokens = True                 # what an engine says whose embedding takes device tokens
        self.fed = {}                                  # request -> running sum of the tokens fed

    def step(self, entries):
        rows = []
        self.steps.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            toks = [int(self.token_feed[-1 - t]) if t < 0 else t for t in e.tokens]
            rc = self.cache.live[e.request_id]
            self.cache.extend(rc, len(toks))
            self.cache.commit(rc, len(toks))
            self.fed[e.request_id] = self.fed.get(e.request_id, 0) + sum(toks)
            for _ in e.want:
                row = torch.zeros(self.vocab)
                row[(self.fed[e.request_id] * 7 + rc.seq_len) % self.vocab] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, self.vocab)

    def end(self, rid):
        super().end(rid)
        self.fed.pop(rid, None)


class LaunchingSampler:
    """launch() leaves the chosen ids in `out` (the feed) and hands them over at collect()."""

    def __init__(self, rows=8):
        self.out = torch.zeros(rows, dtype=torch.int32)
        self.launched = self.collected = 0

    def launch(self, logits, states):
        toks = logits.argmax(-1).to(torch.int32)
        self.out[:len(states)] = toks
        self.launched += 1
        return (toks.tolist(), states)

    def collect(self, handle):
        toks, states = handle
        self.collected += 1
        for s, t in zip(states, toks):
            s.record(t)
        return toks

    def sample(self, logits, states):
        return self.collect(self.launch(logits, states))


def _run_both(add_requests, late=None, **engine_opts):
    outs = []
    for ahead in (False, True):
        eng = FeedingEngine(**engine_opts)
        s = Scheduler(eng, LaunchingSampler(), run_ahead=ahead)
        assert s.run_ahead == ahead
        ids = add_requests(s)
        steps = 0
        while s.has_work():
            s.step()
            steps += 1
            if late is not None and steps == late[0]:
                ids.append(late[1](s))
        assert not eng.cache.live and eng.cache.groups[0].pool.free_pages == engine_opts["pages"]
        outs.append(([s.request(i).output for i in ids], dict(s.stats), eng.steps))
    return outs


def test_running_ahead_gives_the_same_tokens():
    def add(s):
        return [s.add_request([3, 4, 5], 9), s.add_request([6] * 7, 4), s.add_request([1], 12)]

    (want, plain_stats, _), (got, stats, steps) = _run_both(add, pages=32, max_tokens=16)
    assert got == want and all(len(o) == n for o, n in zip(got, (9, 4, 12)))
    assert plain_stats["steps_ahead"] == 0 and stats["steps_ahead"] >= 8
    # a request that ends by its length is left out of the step launched ahead: no row of it is dropped
    assert stats["rows_dropped"] == 0


def test_running_ahead_drops_the_row_of_a_request_stopped_in_mid_flight():
    probe = FeedingEngine(pages=32, max_tokens=16)
    s = Scheduler(probe, LaunchingSampler(), run_ahead=False)
    rid = s.add_request([2, 9, 4], 12)
    free = s.run()[rid]
    at = next(k for k in range(4, 12) if free.index(free[k]) == k)
    stop = free[at]

    def add(s):
        return [s.add_request([2, 9, 4], 12, stop_ids=[stop]), s.add_request([8, 8], 12)]

    (want, _, _), (got, stats, _) = _run_both(add, pages=32, max_tokens=16)
    assert got == want and got[0] == free[:at + 1]
    assert stats["rows_dropped"] == 1


def test_running_ahead_pauses_for_arrivals_and_short_pages():
    def add(s):
        return [s.add_request([1, 2, 3, 4, 5], 14), s.add_request([7, 7, 7], 14)]

    late = (6, lambda s: s.add_request([9, 9, 9, 9], 6))
    (want, _, _), (got, stats, steps) = _run_both(add, late, pages=32, max_tokens=16)
    assert got == want
    # the arrival's prompt went in beside decoded tokens, in a step planned with all tokens at hand
    assert any(any(n > 1 for _, n, _ in st) and any(n == 1 for _, n, _ in st) for st in steps)
    # with pages too few for everybody the ahead path stands back and the push-out logic decides
    (want, plain_stats, _), (got, stats, _) = _run_both(add, pages=8, max_tokens=16)
    assert got == want and stats["pushed_out"] >= 1 and stats["pushed_out"] == plain_stats["pushed_out"]


def test_keys_per_split_of_the_decode_kernel():
    """The choice is a multiple of 64 the kernel takes, short for a lone short sequence (many small
    CTAs), long when there are rounds of CTAs anyway, and the same for the same question."""
    from fastllm_py_b200.native.attention import decode_split_keys, decode_splits

    for n_tokens in (1, 3, 8, 64, 300):
        for kv_heads in (1, 8, 32):
            for longest in (1, 63, 64, 65, 500, 2049, 4096, 100000):
                for head_dim in (16, 128, 256):
                    keys = decode_split_keys(n_tokens, kv_heads, longest, 148, head_dim)
                    assert keys % 64 == 0 and 64 <= keys <= 1024
                    assert decode_splits(longest, keys) * keys >= longest
    assert decode_split_keys(1, 32, 300) <= 128
    assert decode_split_keys(64, 32, 2049) >= 512
    assert decode_split_keys(8, 32, 2304) == decode_split_keys(8, 32, 2304)
