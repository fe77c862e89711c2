"""The cache manager: pages of keys and values with a block table per request,
and slots of fixed size for per-request state.

* Layers whose mixers need the same thing of the cache (every key, or a window of
  w keys; the same heads and head size) form a *group*.  A group has its own pool of
  page ids and every request has one block table per group.
* Pages are handed out lowest id first and reused last-freed first; page 0 of every
  group is never handed out: it is where padded rows of a fixed-shape batch write
  (reference: src/core/block_allocator.cpp:7-35).
* Pages go back when a request is closed (finished or preempted), when a
  reservation cannot be completed (all or nothing), and, in a window group, as soon
  as every key on a page is older than the window of all tokens still to come.
* A request also holds one state slot (an index into per-layer state pools of fixed
  size) from opening to closing, whether or not any layer keeps state.

This module is host code only and holds no tensors; ``storage.py`` owns the memory.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..parts.spec import CacheSpec


class CacheError(RuntimeError):
    pass


class PageAllocator:
    """A fixed pool of page ids with a LIFO free list; ids below ``reserved`` are never given out."""

    def __init__(self, num_pages: int, reserved: int = 1):
        if num_pages <= reserved:
            raise CacheError(f"a pool needs more than {reserved} pages, got {num_pages}")
        self.num_pages = num_pages
        self.reserved = reserved
        self._free = list(range(num_pages - 1, reserved - 1, -1))  # pop() gives the lowest id first
        self._held = [False] * num_pages

    @property
    def num_usable(self) -> int:
        return self.num_pages - self.reserved

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        """A page id, or -1 when none is free."""
        if not self._free:
            return -1
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, pages: Sequence[int]) -> None:
        """Gives pages back; the first of ``pages`` is the next to be handed out again."""
        for p in reversed(list(pages)):
            if p < self.reserved or p >= self.num_pages:
                raise CacheError(f"page id {p} is not a page of this pool")
            if not self._held[p]:
                raise CacheError(f"page {p} freed twice")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]


@dataclass
class GroupInfo:
    """One cache group: its needs, and which cache-owning layer calls belong to it."""

    spec: CacheSpec
    owners: List[int] = field(default_factory=list)   # indices of run-order entries that own a cache

    @property
    def window(self) -> int:
        return self.spec.window if self.spec.kind == "window" else 0


@dataclass
class RequestCache:
    """What one request holds."""

    key: object
    state_slot: int
    tables: List[List[int]]          # per group: page id per block index; 0 once released by a window
    num_tokens: int = 0              # positions for which pages are reserved
    released_upto: List[int] = field(default_factory=list)  # per group: blocks below this index were released


class CacheManager:
    def __init__(self, groups: Sequence[GroupInfo], pages_per_group: Sequence[int], page_size: int,
                 num_state_slots: int):
        if len(groups) != len(pages_per_group):
            raise CacheError("one page count per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        self.allocators = [PageAllocator(n) for n in pages_per_group]
        self._free_slots = list(range(num_state_slots - 1, -1, -1))
        self.num_state_slots = num_state_slots
        self._open: Dict[object, RequestCache] = {}
        self.on_open = None   # called with the RequestCache of every newly opened request

    # ------------------------------------------------------------ requests
    def open(self, key: object) -> RequestCache:
        if key in self._open:
            raise CacheError(f"request {key!r} is already open")
        if not self._free_slots:
            raise CacheError("no free state slot: too many live requests")
        rc = RequestCache(key, self._free_slots.pop(), [[] for _ in self.groups], 0, [0] * len(self.groups))
        self._open[key] = rc
        if self.on_open is not None:
            self.on_open(rc)
        return rc

    def get(self, key: object) -> RequestCache:
        try:
            return self._open[key]
        except KeyError:
            raise CacheError(f"request {key!r} is not open") from None

    def is_open(self, key: object) -> bool:
        return key in self._open

    def close(self, key: object) -> None:
        """Gives back every page and the state slot of the request."""
        rc = self._open.pop(key, None)
        if rc is None:
            raise CacheError(f"request {key!r} is not open")
        for g, table in enumerate(rc.tables):
            live = [p for i, p in enumerate(table) if i >= rc.released_upto[g]]
            self.allocators[g].free(live)
        self._free_slots.append(rc.state_slot)

    def num_open(self) -> int:
        return len(self._open)

    # --------------------------------------------------------------- pages
    def blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, rc: RequestCache, new_len: int) -> List[int]:
        """Pages each group would have to hand out to hold positions < new_len."""
        need = self.blocks_for(new_len)
        return [max(0, need - len(t)) for t in rc.tables]

    def can_reserve(self, rc: RequestCache, new_len: int, keep_free: int = 0) -> bool:
        return all(a.num_free - n >= keep_free
                   for a, n in zip(self.allocators, self.pages_needed(rc, new_len)))

    def reserve(self, rc: RequestCache, new_len: int) -> bool:
        """Makes sure pages exist for positions < new_len in every group.  All or
        nothing: on failure what this call took is given back and False is returned."""
        need = self.blocks_for(new_len)
        taken: List[Tuple[int, int]] = []
        for g, table in enumerate(rc.tables):
            while len(table) < need:
                p = self.allocators[g].allocate()
                if p < 0:
                    for gg, pp in reversed(taken):
                        rc.tables[gg].pop()
                        self.allocators[gg].free([pp])
                    return False
                table.append(p)
                taken.append((g, p))
        rc.num_tokens = max(rc.num_tokens, new_len)
        return True

    def release_passed(self, rc: RequestCache, num_computed: int) -> int:
        """After ``num_computed`` positions are in the cache: in window groups, frees the
        pages whose keys no later token can see (key j is dead when j <= n - window for
        the next position n).  Returns how many pages were freed."""
        freed = 0
        for g, info in enumerate(self.groups):
            w = info.window
            if w <= 0:
                continue
            dead_keys = num_computed - w + 1          # keys 0 .. dead_keys-1 are dead
            dead_blocks = max(0, dead_keys) // self.page_size
            dead_blocks = min(dead_blocks, len(rc.tables[g]))
            if dead_blocks > rc.released_upto[g]:
                pages = rc.tables[g][rc.released_upto[g]:dead_blocks]
                self.allocators[g].free(pages)
                for i in range(rc.released_upto[g], dead_blocks):
                    rc.tables[g][i] = 0
                freed += len(pages)
                rc.released_upto[g] = dead_blocks
        return freed

    def slot(self, rc: RequestCache, group: int, pos: int) -> int:
        """The cache slot (page * page_size + offset) of position ``pos``."""
        return rc.tables[group][pos // self.page_size] * self.page_size + pos % self.page_size

    # ----------------------------------------------------------- inspection
    def num_free_pages(self, group: int = 0) -> int:
        return self.allocators[group].num_free

    def num_total_pages(self, group: int = 0) -> int:
        return self.allocators[group].num_usable

    def check_invariants(self) -> None:
        """No page lost, none held twice: every usable page is either free or in exactly
        one live table entry.  Raises CacheError otherwise (used by the tests)."""
        for g, a in enumerate(self.allocators):
            seen: Dict[int, object] = {}
            for rc in self._open.values():
                for i, p in enumerate(rc.tables[g]):
                    if i < rc.released_upto[g]:
                        continue
                    if p in seen:
                        raise CacheError(f"group {g}: page {p} held by {seen[p]!r} and {rc.key!r}")
                    if not a.is_held(p):
                        raise CacheError(f"group {g}: page {p} of {rc.key!r} is on the free list")
                    seen[p] = rc.key
            if len(seen) + a.num_free != a.num_usable:
                raise CacheError(f"group {g}: {a.num_usable - a.num_free - len(seen)} pages lost")
        slots = [rc.state_slot for rc in self._open.values()]
        if len(set(slots)) != len(slots) or len(slots) + len(self._free_slots) != self.num_state_slots:
            raise CacheError("state slots lost or held twice")
