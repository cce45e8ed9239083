"""CacheManager: pages, block tables and state slots of the live requests.

Owns
  * one PagePool per group of layers with the same need (all keys / a window);
  * for each live request and group, the list of its pages by logical index
    (the block table row; -1 where a window has passed and the page went back);
  * one SlotPool for per-request state of fixed size;
  * the device tensors behind all of it (when given a device).

It replaces fastllm-py's two cache forms: the growable per-sequence buffer
(`KVCache`, fastllm_py/model.py:76-123) and the preallocated
(B, max_len, KVH, D) slot arrays of the batched decoder
(fastllm_py/batched.py:118-121).  Unlike the latter it has bounds: a request
cannot grow past `max_pages_per_request`, and asking for more pages than are
free raises OutOfPages and changes nothing.

Device layout of one layer's cache in a group: [num_pages, *need.page_shape(page_size)];
what a page holds is the need's business (keys and values, `cache.needs.PagedKV`), not
the manager's.

Check mode (`poison`): every page that goes back is overwritten on the device with a
value no computation survives (1e4 by default: keys or values of that size swamp a
softmax or an output row without turning masked places into NaN), so that a kernel which
reads a page it no longer owns, or a place of a fresh page that was never written, shows
in the logits instead of passing by luck.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .needs import FixedState, PagedNeed
from .pages import OutOfPages, PagePool, SlotPool


@dataclass
class PageGroup:
    need: PagedNeed
    cache_ids: list
    pool: PagePool
    tensors: dict = field(default_factory=dict)      # cache id -> device tensor

    @property
    def window(self):
        return self.need.window


@dataclass
class RequestCache:
    """What one live request holds."""
    request_id: object
    slot: int
    seq_len: int = 0                                  # tokens whose keys/values are written
    reserved: int = 0                                 # tokens that the pages taken so far can hold
    pages: list = field(default_factory=list)         # per group: list of page ids by logical index (-1: given back)
    released: list = field(default_factory=list)      # per group: logical pages below this index went back
    tables: list = field(default_factory=list)        # per group: the same as `pages`, as an int32 row of fixed width
    version: int = 0                                  # bumped whenever a table row changes
    uid: int = 0                                      # unique over the manager's life (request ids may be reused)


class CacheManager:
    def __init__(self, needs: dict, page_size: int, num_pages: int, max_requests: int,
                 max_pages_per_request: int, poison: float | None = None):
        """`needs`: cache id -> PagedNeed | FixedState | None, one per run that has a cache."""
        self.page_size = page_size
        self.poison = poison                          # check mode: returned pages are filled with this
        self.pages_poisoned = 0
        self.max_requests = max_requests
        self.max_pages_per_request = max_pages_per_request
        self.groups: list[PageGroup] = []
        self.group_of: dict = {}                      # cache id -> index into groups
        self.state_needs: dict = {}                   # cache id -> FixedState
        self.state_tensors: dict = {}
        by_need: dict = {}
        for cid, need in needs.items():
            if need is None:
                continue
            if isinstance(need, FixedState):
                self.state_needs[cid] = need
            elif isinstance(need, PagedNeed):
                if need not in by_need:
                    by_need[need] = len(self.groups)
                    self.groups.append(PageGroup(need, [], PagePool(num_pages)))
                g = by_need[need]
                self.groups[g].cache_ids.append(cid)
                self.group_of[cid] = g
            else:
                raise TypeError(f"cache {cid}: unknown need {need!r}")
        self.slots = SlotPool(max_requests)
        self.live: dict = {}                          # request id -> RequestCache
        self._next_uid = 1

    # ------------------------------------------------------------ device side
    def allocate(self, device, activation_dtype):
        """Create the device tensors (pages of every layer, state rows)."""
        import torch

        for g in self.groups:
            dt = activation_dtype if g.need.dtype == "activation" else getattr(torch, g.need.dtype)
            shape = (g.pool.num_pages,) + tuple(g.need.page_shape(self.page_size))
            for cid in g.cache_ids:
                g.tensors[cid] = torch.zeros(shape, dtype=dt, device=device)
                if self.poison is not None:
                    g.tensors[cid].fill_(self.poison)     # never-written places are as bad as stale ones
        for cid, need in self.state_needs.items():
            dt = activation_dtype if need.dtype == "activation" else getattr(torch, need.dtype)
            self.state_tensors[cid] = torch.zeros((self.max_requests,) + tuple(need.shape),
                                                  dtype=dt, device=device)

    @staticmethod
    def bytes_per_token(needs: dict, page_size: int, itemsize: int) -> int:
        """Cache bytes one token costs over all paged layers (for sizing the pools)."""
        return sum(need.bytes_per_token(page_size, itemsize) for need in needs.values()
                   if isinstance(need, PagedNeed))

    def _give_back(self, group: PageGroup, pages: list) -> None:
        """Pages return to the group's pool; in check mode their contents are destroyed first
        (on the current stream, so after every kernel launched so far that may still read them)."""
        if not pages:
            return
        if self.poison is not None and group.tensors:
            import torch

            any_tensor = next(iter(group.tensors.values()))
            index = torch.tensor(pages, dtype=torch.long, device=any_tensor.device)
            for tensor in group.tensors.values():
                tensor.index_fill_(0, index, self.poison)
            self.pages_poisoned += len(pages)
        group.pool.give_back(pages)

    # ------------------------------------------------------------- requests
    def admit(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise RuntimeError(f"request {request_id!r} is already live")
        slot = self.slots.take()
        rc = RequestCache(request_id, slot, pages=[[] for _ in self.groups],
                          released=[0] * len(self.groups),
                          tables=[np.full(self.max_pages_per_request, -1, dtype=np.int32)
                                  for _ in self.groups], uid=self._next_uid)
        self._next_uid += 1
        self.live[request_id] = rc
        return rc

    def _pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def pages_missing(self, rc: RequestCache, new_tokens: int) -> int:
        """Pages each group must still take so that `new_tokens` more tokens fit."""
        return max(0, self._pages_for(rc.seq_len + new_tokens) - self._pages_for(rc.reserved))

    def can_extend(self, rc: RequestCache, new_tokens: int, spare: int = 0) -> bool:
        """True if extend() would succeed and leave `spare` pages free in every group."""
        if self._pages_for(rc.seq_len + new_tokens) > self.max_pages_per_request:
            return False
        missing = self.pages_missing(rc, new_tokens)
        return all(g.pool.free_pages >= missing + spare for g in self.groups)

    def extend(self, rc: RequestCache, new_tokens: int) -> None:
        """Take the pages for `new_tokens` more tokens in every group, or raise
        OutOfPages and take none."""
        total = self._pages_for(rc.seq_len + new_tokens)
        if total > self.max_pages_per_request:
            raise OutOfPages(
                f"request {rc.request_id!r} would hold {rc.seq_len + new_tokens} tokens; "
                f"the most a request may hold is {self.max_pages_per_request * self.page_size}")
        missing = self.pages_missing(rc, new_tokens)
        if missing == 0:
            return
        for g in self.groups:
            if g.pool.free_pages < missing:
                raise OutOfPages(
                    f"request {rc.request_id!r} needs {missing} more pages, "
                    f"{g.pool.free_pages} free of {g.pool.num_pages}")
        for gi, g in enumerate(self.groups):
            have = len(rc.pages[gi])
            new = g.pool.take(missing)
            rc.pages[gi].extend(new)
            rc.tables[gi][have:have + missing] = new
        rc.version += 1
        rc.reserved = total * self.page_size

    def commit(self, rc: RequestCache, new_tokens: int) -> None:
        """The step wrote `new_tokens` tokens.  Pages that a window has passed go back."""
        rc.seq_len += new_tokens
        if rc.seq_len > rc.reserved:
            raise RuntimeError(f"request {rc.request_id!r}: {rc.seq_len} tokens written, "
                               f"pages for {rc.reserved}")
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            # The next query sits at position seq_len and sees keys from
            # seq_len - window + 1 on; pages wholly below that are dead.
            first_needed = rc.seq_len - g.window + 1
            row = rc.pages[gi]
            dead_pages = min(max(0, first_needed) // self.page_size, len(row))
            if dead_pages > rc.released[gi]:
                self._give_back(g, row[rc.released[gi]:dead_pages])
                for i in range(rc.released[gi], dead_pages):
                    row[i] = -1
                rc.tables[gi][rc.released[gi]:dead_pages] = -1
                rc.version += 1
                rc.released[gi] = dead_pages

    def release(self, request_id) -> None:
        """The request ended (or is pushed out): everything it holds goes back."""
        rc = self.live.pop(request_id)
        for gi, g in enumerate(self.groups):
            self._give_back(g, [p for p in rc.pages[gi] if p >= 0])
            rc.pages[gi] = []
        self.slots.give_back(rc.slot)

    # ------------------------------------------------------ tables for a step
    def block_table_row(self, group: int, rc: RequestCache, out: np.ndarray) -> None:
        out[:] = rc.tables[group]

    def slot_mapping(self, group: int, rc: RequestCache, count: int, out: np.ndarray) -> None:
        """Where the next `count` tokens of the request go: page * page_size + offset."""
        ps = self.page_size
        if count == 1:
            page = int(rc.tables[group][rc.seq_len // ps])
            if page < 0:
                raise RuntimeError(f"request {rc.request_id!r}: writing into a page that was given back")
            out[0] = page * ps + rc.seq_len % ps
            return
        pos = np.arange(rc.seq_len, rc.seq_len + count)
        pages = rc.tables[group][pos // ps]
        if (pages < 0).any():
            raise RuntimeError(f"request {rc.request_id!r}: writing into a page that was given back")
        out[:count] = pages * ps + pos % ps

    # ------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, none held twice: the pools' books equal the requests'."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = []
            for rc in self.live.values():
                held.extend(p for p in rc.pages[gi] if p >= 0)
            if len(held) != len(set(held)):
                raise AssertionError(f"group {gi}: a page is held by two requests")
            if len(held) != g.pool.held_pages:
                raise AssertionError(
                    f"group {gi}: requests hold {len(held)} pages, pool says {g.pool.held_pages}")
        slots = [rc.slot for rc in self.live.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("a slot is held by two requests")
        if len(slots) != self.max_requests - self.slots.free_slots:
            raise AssertionError("slot pool and live requests disagree")
