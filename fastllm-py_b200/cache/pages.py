"""PagePool: fixed-size pages of a cache, handed out and taken back.

fastllm-py never returns cache memory: every slot owns `max_len` rows for the
whole run (fastllm_py/batched.py:118-121) and a finished slot is only marked
empty (batched.py:366).  Here pages go back to a free list the moment their
owner ends (or a window has passed them) and the next request takes them.

The pool checks its own books: a page is either free or held by exactly one
owner, and giving back a page that is not held is an error, not a no-op.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """The pool cannot serve the pages asked for; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        # Lowest page first, so that page use is reproducible.
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def held_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, count: int) -> list:
        """`count` pages, or OutOfPages with the pool unchanged."""
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages asked for, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(count)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise RuntimeError(f"page {p} given back twice (or never taken)")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.num_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p}: held={self._held[p]} free={p in free}")


class SlotPool:
    """Slots for per-request state of fixed size (one per live request).

    fastllm-py's counterpart is the slot index of the batched decoder, which
    owns `pos[b]`, the last token and the KV rows (batched.py:117, :351-352).
    Here a slot owns only what has a fixed size per request: a row in every
    state tensor that a mixer asked for."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_slots} request slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise RuntimeError(f"slot {slot} given back twice (or never taken)")
        self._held[slot] = False
        self._free.append(slot)
