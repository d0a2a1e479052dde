"""Host-side bookkeeping of cache pages, block tables and per-request state slots.

The reference's ``KVCacheManager`` (csrc/scheduler/kv_cache_manager.h:31-95) keeps one pool of blocks:
``allocate_slots`` takes ``ceil((computed + n) / block_size) − held`` blocks all-or-nothing
(kv_cache_manager.cpp:232-263), freed blocks go to the tail of a free list and are taken from its head
(:45-98), and a request's blocks are released when it finishes, is aborted or is preempted (:265-287).

Here the same rules hold per *cache group*.  A group is a set of layer runs with one page shape and one
retention rule — all tokens, or a window of the last ``w`` — and has a pool and block tables of its own;
a page id addresses the same token range in every run of its group.  An allocation succeeds in all
groups or in none.  After a step, pages that a windowed group's next query can no longer see are given
back at once and their block-table entry becomes -1.  Beside the pages, every request holds one slot
of fixed-size state from a second pool, taken at admission and released with the pages.

Page ids and slots are plain integers; device memory is owned by ``cache/storage.py``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence


class CacheError(RuntimeError):
    """A misuse of the cache manager (unknown request, double admit, double free)."""


@dataclass(frozen=True)
class CacheGroupSpec:
    """One group of layer runs sharing a page shape and a retention rule."""

    runs: tuple[int, ...]
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every token is kept

    def key(self) -> tuple:
        return (self.num_kv_heads, self.head_dim, self.window)


class PagePool:
    """``num_pages`` page ids with a FIFO free list: freed pages go to the tail, allocations take from the head."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: Deque[int] = deque(range(num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise CacheError("cannot take a negative number of pages")
        if n > len(self._free):
            return None
        pages = [self._free.popleft() for _ in range(n)]
        for p in pages:
            self._held[p] = True
        return pages

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise CacheError(f"page {p} is not in this pool of {self.num_pages}")
            if not self._held[p]:
                raise CacheError(f"page {p} is freed twice")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free exactly once or held."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            if self._held[p] == (p in set(free)):
                raise CacheError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class SlotPool:
    """Slots of fixed-size per-request state; the lowest free slot is taken first."""

    def __init__(self, num_slots: int) -> None:
        if num_slots <= 0:
            raise CacheError("a slot pool needs at least one slot")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheError(f"state slot {slot} is freed twice or was never taken")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


@dataclass
class _Held:
    slot: int
    serial: int = 0                                             # number of this admission; never handed out twice
    num_tokens: int = 0                                         # tokens whose keys/values are stored
    tables: List[List[int]] = field(default_factory=list)       # per group: page of every page index, -1 if given back
    first_live: List[int] = field(default_factory=list)         # per group: first page index still held


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroupSpec], page_size: int, num_pages: int | Sequence[int],
                 max_requests: int) -> None:
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise CacheError("one page count per group")
        self.pools = [PagePool(n) for n in counts]
        self.slots = SlotPool(max_requests)
        self._held: Dict[Hashable, _Held] = {}
        self._admissions = 0
        self.newly_admitted: List[int] = []   # slots whose state must be zeroed before the next step

    # ---- queries ---------------------------------------------------------------------------------
    def __contains__(self, request_id: Hashable) -> bool:
        return request_id in self._held

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def num_tokens(self, request_id: Hashable) -> int:
        return self._get(request_id).num_tokens

    def slot(self, request_id: Hashable) -> int:
        return self._get(request_id).slot

    def serial(self, request_id: Hashable) -> int:
        """The number of the admission under which the request holds its pages.  A request id that comes back
        after its release (a caller's conversation id, a preempted request) gets a new one, so anything cached per
        request outside the manager — block-table rows already on the device — can tell the two apart."""
        return self._get(request_id).serial

    def block_table(self, request_id: Hashable, group: int = 0) -> List[int]:
        """Page of every page index of the request in ``group``; -1 where the page was given back."""
        return self._get(request_id).tables[group]

    def live_requests(self) -> List[Hashable]:
        return list(self._held)

    def _get(self, request_id: Hashable) -> _Held:
        try:
            return self._held[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} holds nothing in the cache") from None

    def _pages_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, request_id: Hashable, num_new_tokens: int) -> List[int]:
        """Per group, how many more pages ``num_new_tokens`` further tokens need."""
        held = self._held.get(request_id)
        have = held.num_tokens if held else 0
        need = self._pages_for(have + num_new_tokens)
        return [need - (len(held.tables[g]) if held else 0) for g in range(len(self.groups))]

    # ---- life of a request ---------------------------------------------------------------------------
    def admit(self, request_id: Hashable) -> Optional[int]:
        """Give the request a state slot and empty block tables; None if no slot is free."""
        if request_id in self._held:
            raise CacheError(f"request {request_id!r} is already admitted")
        slot = self.slots.take()
        if slot is None:
            return None
        n = len(self.groups)
        self._admissions += 1
        self._held[request_id] = _Held(slot=slot, serial=self._admissions, tables=[[] for _ in range(n)],
                                       first_live=[0] * n)
        self.newly_admitted.append(slot)
        return slot

    def allocate(self, request_id: Hashable, num_new_tokens: int) -> bool:
        """Pages for ``num_new_tokens`` more tokens in every group, or nothing at all."""
        if num_new_tokens < 0:
            raise CacheError("cannot allocate for a negative number of tokens")
        held = self._get(request_id)
        need = self.pages_needed(request_id, num_new_tokens)
        if any(n > self.pools[g].num_free for g, n in enumerate(need)):
            return False
        for g, n in enumerate(need):
            if n > 0:
                held.tables[g].extend(self.pools[g].take(n))
        return True

    def commit(self, request_id: Hashable, num_new_tokens: int) -> None:
        """Record that a step stored ``num_new_tokens`` more tokens; give back pages a window has passed."""
        held = self._get(request_id)
        total = held.num_tokens + num_new_tokens
        if num_new_tokens < 0:
            raise CacheError("cannot commit a negative number of tokens")
        for table in held.tables:
            if self._pages_for(total) > len(table):
                raise CacheError(f"request {request_id!r}: {total} tokens do not fit the pages it holds")
        held.num_tokens = total
        for g, spec in enumerate(self.groups):
            if spec.window is None:
                continue
            # the next query sits at position >= total and sees keys > total - window
            first_needed = max(0, total - spec.window + 1)
            first_page = first_needed // self.page_size
            table = held.tables[g]
            gone = []
            for idx in range(held.first_live[g], min(first_page, len(table))):
                if table[idx] >= 0:
                    gone.append(table[idx])
                    table[idx] = -1
            if gone:
                self.pools[g].give_back(gone)
            held.first_live[g] = max(held.first_live[g], min(first_page, len(table)))

    def release(self, request_id: Hashable) -> None:
        """Give back everything the request holds (finish, abort or preemption)."""
        held = self._get(request_id)
        for g, table in enumerate(held.tables):
            self.pools[g].give_back([p for p in table if p >= 0])
        self.slots.give_back(held.slot)
        if held.slot in self.newly_admitted:
            self.newly_admitted.remove(held.slot)
        del self._held[request_id]

    def take_newly_admitted(self) -> List[int]:
        out, self.newly_admitted = self.newly_admitted, []
        return out

    # ---- addressing for a step -------------------------------------------------------------------------
    def slot_mapping(self, request_id: Hashable, group: int, start: int, count: int) -> List[int]:
        """``page * page_size + offset`` of the tokens at positions ``start .. start+count-1``."""
        table = self._get(request_id).tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + count):
            idx = pos // ps
            if idx >= len(table) or table[idx] < 0:
                raise CacheError(f"request {request_id!r}: position {pos} has no page in group {group}")
            out.append(table[idx] * ps + pos % ps)
        return out

    def check(self) -> None:
        """No page lost, held twice or freed twice; every slot accounted for."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen = set()
            for rid, held in self._held.items():
                for p in held.tables[g]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"page {p} of group {g} is held twice")
                    seen.add(p)
            if len(seen) + pool.num_free != pool.num_pages:
                raise CacheError(f"group {g}: {pool.num_pages - len(seen) - pool.num_free} pages are lost")
        slots = [h.slot for h in self._held.values()]
        if len(set(slots)) != len(slots) or len(slots) + self.slots.num_free != self.slots.num_slots:
            raise CacheError("state slots are lost or held twice")


def group_runs(needs: Dict[int, "object"]) -> List[CacheGroupSpec]:
    """Group runs by (kv heads, head size, window): runs with equal needs share pages ids and tables."""
    by_key: Dict[tuple, List[int]] = {}
    for run in sorted(needs):
        n = needs[run]
        by_key.setdefault((n.num_kv_heads, n.head_dim, n.window), []).append(run)
    return [CacheGroupSpec(tuple(runs), k[0], k[1], k[2]) for k, runs in by_key.items()]
