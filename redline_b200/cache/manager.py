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

The state lives in the native host core (``csrc/host_core.cpp``, bound by ``native.py``);
the classes here are its Python face.  This module is host code only and holds no
tensors; ``storage.py`` owns the memory.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_int, c_int32
from dataclasses import dataclass, field
from typing import Dict, List, Sequence

from ..parts.spec import CacheSpec
from . import native


class CacheError(RuntimeError):
    pass


def _i32_array(values: Sequence[int]):
    return (c_int32 * max(len(values), 1))(*values)


def _raise_free_error(code: int, bad: int) -> None:
    if code == -1:
        raise CacheError(f"page id {bad} is not a page of this pool")
    if code == -2:
        raise CacheError(f"page {bad} freed twice")
    raise CacheError(f"page pool error {code}")


class PageAllocator:
    """A fixed pool of page ids with a LIFO free list; ids below ``reserved`` are never given out."""

    def __init__(self, num_pages: int, reserved: int = 1):
        if num_pages <= reserved:
            raise CacheError(f"a pool needs more than {reserved} pages, got {num_pages}")
        self._lib = native.lib()
        self._h = self._lib.rl_pool_create(num_pages, reserved)
        if not self._h:
            raise CacheError("the page pool could not be created")
        self.num_pages = num_pages
        self.reserved = reserved

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rl_pool_destroy(h)

    @property
    def num_usable(self) -> int:
        return self._lib.rl_pool_num_usable(self._h)

    @property
    def num_free(self) -> int:
        return self._lib.rl_pool_num_free(self._h)

    def allocate(self) -> int:
        """A page id, or -1 when none is free."""
        return self._lib.rl_pool_allocate(self._h)

    def free(self, pages: Sequence[int]) -> None:
        """Gives pages back; the first of ``pages`` is the next to be handed out again."""
        pages = list(pages)
        bad = c_int(0)
        code = self._lib.rl_pool_free(self._h, _i32_array(pages), len(pages), byref(bad))
        if code < 0:
            _raise_free_error(code, bad.value)

    def is_held(self, page: int) -> bool:
        return bool(self._lib.rl_pool_is_held(self._h, page))


@dataclass
class GroupInfo:
    """One cache group: its needs, and which cache-owning layer calls belong to it."""

    spec: CacheSpec
    owners: List[int] = field(default_factory=list)   # indices of run-order entries that own a cache

    @property
    def window(self) -> int:
        return self.spec.window if self.spec.kind == "window" else 0


class RequestCache:
    """What one request holds: a state slot and, per group, a block table (page id per block index; 0
    once released by a window).  The tables live in the native core; ``tables`` copies them out."""

    __slots__ = ("key", "rid", "state_slot", "_m")

    def __init__(self, key: object, rid: int, state_slot: int, manager: "CacheManager"):
        self.key = key
        self.rid = rid
        self.state_slot = state_slot
        self._m = manager

    def table(self, group: int) -> List[int]:
        ptr = POINTER(c_int32)()
        n = self._m._lib.rl_hc_table(self._m._h, self.rid, group, byref(ptr))
        if n < 0:
            raise CacheError(f"request {self.key!r} is not open")
        return ptr[:n]

    @property
    def tables(self) -> List[List[int]]:
        return [self.table(g) for g in range(len(self._m.groups))]

    @property
    def num_tokens(self) -> int:
        """Positions for which pages are reserved."""
        return self._m._lib.rl_hc_num_tokens(self._m._h, self.rid)

    @property
    def released_upto(self) -> List[int]:
        """Per group: blocks below this index were released."""
        return [self._m._lib.rl_hc_released_upto(self._m._h, self.rid, g) for g in range(len(self._m.groups))]


class CacheManager:
    def __init__(self, groups: Sequence[GroupInfo], pages_per_group: Sequence[int], page_size: int,
                 num_state_slots: int):
        if len(groups) != len(pages_per_group):
            raise CacheError("one page count per group is needed")
        for n in pages_per_group:
            if n <= 1:
                raise CacheError(f"a pool needs more than 1 pages, got {n}")
        self.groups = list(groups)
        self.page_size = page_size
        self.num_state_slots = num_state_slots
        self._lib = native.lib()
        self._h = self._lib.rl_hc_create(len(self.groups), _i32_array(list(pages_per_group)),
                                         _i32_array([g.window for g in self.groups]), page_size, num_state_slots)
        if not self._h:
            raise CacheError("the cache manager could not be created")
        self._open: Dict[object, RequestCache] = {}
        self.on_open = None   # called with the RequestCache of every newly opened request

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rl_hc_destroy(h)

    # ------------------------------------------------------------ requests
    def open(self, key: object) -> RequestCache:
        if key in self._open:
            raise CacheError(f"request {key!r} is already open")
        rid = self._lib.rl_hc_open(self._h)
        if rid < 0:
            raise CacheError("no free state slot: too many live requests")
        rc = RequestCache(key, rid, self._lib.rl_hc_state_slot(self._h, rid), self)
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
        bad = c_int(0)
        code = self._lib.rl_hc_close(self._h, rc.rid, byref(bad))
        if code < 0:
            _raise_free_error(code, bad.value)

    def adopt(self, key: object, rid: int) -> RequestCache:
        """The face of a request that native code (the scheduler's planner) has opened in the core."""
        if key in self._open:
            raise CacheError(f"request {key!r} is already open")
        rc = RequestCache(key, rid, self._lib.rl_hc_state_slot(self._h, rid), self)
        self._open[key] = rc
        if self.on_open is not None:
            self.on_open(rc)
        return rc

    def forget(self, key: object) -> None:
        """Drops the face of a request that native code has already closed in the core."""
        if self._open.pop(key, None) is None:
            raise CacheError(f"request {key!r} is not open")

    def num_open(self) -> int:
        return len(self._open)

    # --------------------------------------------------------------- pages
    def blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, rc: RequestCache, new_len: int) -> List[int]:
        """Pages each group would have to hand out to hold positions < new_len."""
        need = self.blocks_for(new_len)
        ptr = POINTER(c_int32)()
        return [max(0, need - self._lib.rl_hc_table(self._h, rc.rid, g, byref(ptr))) for g in range(len(self.groups))]

    def can_reserve(self, rc: RequestCache, new_len: int, keep_free: int = 0) -> bool:
        return all(self.num_free_pages(g) - n >= keep_free for g, n in enumerate(self.pages_needed(rc, new_len)))

    def reserve(self, rc: RequestCache, new_len: int) -> bool:
        """Makes sure pages exist for positions < new_len in every group.  All or
        nothing: on failure what this call took is given back and False is returned."""
        code = self._lib.rl_hc_reserve(self._h, rc.rid, new_len)
        if code < 0:
            raise CacheError(f"request {rc.key!r} is not open")
        return code == 1

    def release_passed(self, rc: RequestCache, num_computed: int) -> int:
        """After ``num_computed`` positions are in the cache: in window groups, frees the
        pages whose keys no later token can see (key j is dead when j <= n - window for
        the next position n).  Returns how many pages were freed."""
        n = self._lib.rl_hc_release_passed(self._h, rc.rid, num_computed)
        if n < 0:
            raise CacheError(f"request {rc.key!r}: releasing pages failed ({n})")
        return n

    def slot(self, rc: RequestCache, group: int, pos: int) -> int:
        """The cache slot (page * page_size + offset) of position ``pos``."""
        return rc.table(group)[pos // self.page_size] * self.page_size + pos % self.page_size

    # ----------------------------------------------------------- inspection
    def num_free_pages(self, group: int = 0) -> int:
        return self._lib.rl_hc_num_free(self._h, group)

    def num_total_pages(self, group: int = 0) -> int:
        return self._lib.rl_hc_num_usable(self._h, group)

    def check_invariants(self) -> None:
        """No page lost, none held twice: every usable page is either free or in exactly
        one live table entry.  Raises CacheError otherwise (used by the tests)."""
        buf = ctypes.create_string_buffer(256)
        if self._lib.rl_hc_check(self._h, buf, 256):
            raise CacheError(buf.value.decode())
        if self._lib.rl_hc_num_open(self._h) != len(self._open):
            raise CacheError("open requests of the core and of its Python face differ")
