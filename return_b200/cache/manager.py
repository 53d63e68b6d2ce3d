"""The cache manager: pages of keys and values with a block table per request, and slots of
fixed size for per-request state.  Host code only; the device pools live in
``return_b200/cache/storage.py``.

What the reference does (rollout/cache.py:8-162): pages of 64 token slots, one page id
addresses a slab in every layer's K and V pool, a LIFO free list (alloc pops the tail, free
appends), per-session page lists, ``KVCapacityError`` when the free list is too short, and,
for other architectures, ``LinearStateCache`` slots of fixed size per resident session
(rollout/cache.py:340-472).  What is different here:

* Layers are put into **groups** by what they need.  A group of full-attention layers keeps
  every key; a group of sliding-window layers keeps a window of them.  Each group has pages of
  its own (its own pool, free list and block tables), because a window group gives pages back
  while a request is still running and a full group does not.
* Only the last page of a request is partly filled, so a block table is a list of page ids
  indexed by ``position // page_size``; ``-1`` marks a block that the window has passed and
  whose page went back to the pool.
* Every request holds one **slot** (0 .. max_requests-1) for its fixed-size state and as its
  row in device-side tables, whether or not the architecture has such state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence


class KVCapacityError(MemoryError):
    """Pages (or request slots) ran out.  Same name as the reference's error (rollout/engine.py:9-10)."""


@dataclass(frozen=True)
class GroupSpec:
    """What one group of cache layers needs.  ``window`` None: all keys; else the last ``window`` keys."""
    name: str
    page_size: int
    num_pages: int
    window: Optional[int] = None


class PagePool:
    """Free list of one group's pages.  LIFO: the page freed last is handed out first
    (rollout/cache.py:98,153), so reuse shows up early in tests."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))     # page 0 is handed out first
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise KVCapacityError(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            assert not self._held[p], f"page {p} handed out twice"
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise AssertionError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)

    def held_pages(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


@dataclass
class _RequestState:
    slot: int
    length: int = 0                                     # tokens whose keys are (or were) cached
    blocks: List[List[int]] = field(default_factory=list)   # per group: page id per block, -1 = released


class CacheManager:
    """Pages per group and slots per request.

    ``add(rid)`` gives a request a slot; ``append(rid, n)`` makes room for its next ``n`` tokens in
    every group (all or nothing) after giving back what the windows have passed; ``free(rid)``
    returns everything.  Nothing here touches the GPU.
    """

    def __init__(self, groups: Sequence[GroupSpec], max_requests: int):
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.groups = list(groups)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.max_requests = max_requests
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._req: Dict[Hashable, _RequestState] = {}
        # False when something beside the pages depends on every token a request has run (per-request state on the
        # device): a request's length can then not be taken back
        self.truncatable = True
        # called with the slot whenever a request takes one: whoever keeps per-request state on the device
        # starts the slot from zero here, so that every way of admitting a request (replay, scheduler,
        # re-admission after a preemption) resets it
        self.on_slot_taken: List[Callable[[int], None]] = []

    # ------------------------------------------------------------------ requests and slots
    def __contains__(self, rid) -> bool:
        return rid in self._req

    @property
    def num_requests(self) -> int:
        return len(self._req)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def add(self, rid) -> int:
        if rid in self._req:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise KVCapacityError(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        self._req[rid] = _RequestState(slot=slot, blocks=[[] for _ in self.groups])
        for hook in self.on_slot_taken:
            hook(slot)
        return slot

    def free(self, rid) -> None:
        st = self._req.pop(rid)
        for pool, blocks in zip(self.pools, st.blocks):
            pool.give_back([p for p in blocks if p >= 0])
        self._free_slots.append(st.slot)

    def slot(self, rid) -> int:
        return self._req[rid].slot

    def length(self, rid) -> int:
        return self._req[rid].length

    def block_table(self, rid, group: int) -> List[int]:
        return self._req[rid].blocks[group]

    def live(self) -> List[Hashable]:
        return list(self._req)

    # ------------------------------------------------------------------ pages
    def _first_needed_block(self, g: GroupSpec, length: int) -> int:
        """Blocks below this index hold only keys that no query at position >= length can see."""
        if g.window is None:
            return 0
        return max(0, length - g.window + 1) // g.page_size

    def pages_needed(self, rid, n_tokens: int) -> List[int]:
        """Per group: pages that ``append(rid, n_tokens)`` would take beyond those it gives back."""
        st = self._req[rid]
        out = []
        for g, blocks in zip(self.groups, st.blocks):
            end_blocks = (st.length + n_tokens + g.page_size - 1) // g.page_size
            new = max(0, end_blocks - len(blocks))
            first = self._first_needed_block(g, st.length)
            released = sum(1 for b in range(min(first, len(blocks))) if blocks[b] >= 0)
            out.append(new - released)
        return out

    def fits(self, rid, n_tokens: int) -> bool:
        return all(need <= pool.num_free for need, pool in zip(self.pages_needed(rid, n_tokens), self.pools))

    def fits_all(self, rids: Sequence[Hashable], n_tokens: int) -> bool:
        """Whether every one of ``rids`` can append ``n_tokens`` in the same step: their needs are summed per
        group before they are set against the free pages (two requests that each need the last free page
        do not both fit, although ``fits`` says yes to either alone)."""
        total = [0] * len(self.groups)
        for rid in rids:
            for g, need in enumerate(self.pages_needed(rid, n_tokens)):
                total[g] += max(need, 0)     # pages a window gives back are not lent to a request that appends earlier
        return all(need <= pool.num_free for need, pool in zip(total, self.pools))

    def append(self, rid, n_tokens: int) -> int:
        """Room for the next ``n_tokens`` of ``rid`` in every group; returns the old length.

        Raises KVCapacityError and changes nothing if any group lacks the pages."""
        if n_tokens <= 0:
            raise ValueError("append needs at least one token")
        st = self._req[rid]
        if not self.fits(rid, n_tokens):
            short = [(g.name, need, pool.num_free)
                     for g, need, pool in zip(self.groups, self.pages_needed(rid, n_tokens), self.pools)
                     if need > pool.num_free]
            raise KVCapacityError(f"request {rid!r}: pages (group, needed, free) {short}")
        for g, pool, blocks in zip(self.groups, self.pools, st.blocks):
            first = self._first_needed_block(g, st.length)
            gone = [b for b in range(min(first, len(blocks))) if blocks[b] >= 0]
            if gone:
                pool.give_back([blocks[b] for b in gone])
                for b in gone:
                    blocks[b] = -1
            end_blocks = (st.length + n_tokens + g.page_size - 1) // g.page_size
            if end_blocks > len(blocks):
                blocks.extend(pool.take(end_blocks - len(blocks)))
        old = st.length
        st.length += n_tokens
        return old

    def truncate(self, rid, length: int) -> None:
        """Takes the last tokens of a request back: its length becomes ``length`` (not more than it is) and the
        pages behind it return to their pools.  What lies in the kept pages beyond ``length`` is overwritten by
        the tokens that come next."""
        st = self._req[rid]
        if not (0 <= length <= st.length):
            raise ValueError(f"request {rid!r} holds {st.length} tokens; cannot truncate to {length}")
        if length < st.length and not self.truncatable:
            raise ValueError("per-request state depends on the tokens that were run: nothing can be taken back")
        for g, pool, blocks in zip(self.groups, self.pools, st.blocks):
            keep = (length + g.page_size - 1) // g.page_size
            gone = [p for p in blocks[keep:] if p >= 0]
            if gone:
                pool.give_back(gone)
            del blocks[keep:]
        st.length = length

    # ------------------------------------------------------------------ accounting, for tests and stats
    def pages_used(self) -> List[int]:
        return [pool.num_pages - pool.num_free for pool in self.pools]

    def check(self) -> None:
        """No page lost, none held twice, none both free and held; slots likewise."""
        for gi, pool in enumerate(self.pools):
            owned: List[int] = []
            for st in self._req.values():
                owned.extend(p for p in st.blocks[gi] if p >= 0)
            assert len(owned) == len(set(owned)), f"group {gi}: a page is held by two block tables"
            assert sorted(owned) == pool.held_pages(), f"group {gi}: held pages and block tables disagree"
            free = list(pool._free)
            assert len(free) == len(set(free)), f"group {gi}: a page is on the free list twice"
            assert not set(free) & set(owned), f"group {gi}: a page is both free and held"
            assert len(free) + len(owned) == pool.num_pages, f"group {gi}: a page was lost"
        slots = [st.slot for st in self._req.values()]
        assert len(slots) == len(set(slots)), "a slot is held by two requests"
        assert sorted(slots + self._free_slots) == list(range(self.max_requests)), "a slot was lost"
