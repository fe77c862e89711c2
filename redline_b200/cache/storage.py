"""Device memory of the cache: per group ONE allocation, zero-filled once and cut into, for every
layer call that owns a cache and every tensor its mixer caches, a view
[pages, *leading axes, page_size, last axis] (for attention: K and V
[pages, heads, page_size, head_dim], so that a (page, head) is one contiguous
[page_size, head_dim] box); and per state-keeping layer call one pool [slots, *state shape]
(reference layout of the pages: src/cuda/model/kv_cache.cpp:17-52, src/cuda/kernels/kernels.h:15-27)."""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import LayerCache
from ..parts.spec import StateSpec
from .manager import GroupInfo


def bytes_per_page(groups: Sequence[GroupInfo], page_size: int, elem_size: int) -> List[int]:
    return [len(g.owners) * g.spec.elements_per_token() * page_size * elem_size for g in groups]


class CacheStorage:
    def __init__(self, groups: Sequence[GroupInfo], pages_per_group: Sequence[int], page_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.page_size = page_size
        self.pools: List[torch.Tensor] = []
        self._by_owner: Dict[int, LayerCache] = {}
        for gi, (g, n) in enumerate(zip(groups, pages_per_group)):
            per_owner = n * page_size * g.spec.elements_per_token()
            pool = torch.zeros(max(len(g.owners), 1) * per_owner, dtype=dtype, device=device)
            self.pools.append(pool)
            for j, owner in enumerate(g.owners):
                views: Dict[str, torch.Tensor] = {}
                off = j * per_owner
                for t in g.spec.tensors:
                    size = n * page_size * t.elements()
                    views[t.name] = pool[off:off + size].view((n,) + tuple(t.shape[:-1]) + (page_size, t.shape[-1]))
                    off += size
                self._by_owner[owner] = LayerCache(gi, views, True)

    def of_owner(self, owner: int, write: bool) -> LayerCache:
        c = self._by_owner[owner]
        return c if write else LayerCache(c.group, c.tensors, False)

    def nbytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools)


class StateStorage:
    """Pools of fixed-size per-request state, one per layer call that keeps state."""

    def __init__(self, specs: Dict[int, StateSpec], num_slots: int, device: torch.device):
        self.pools: Dict[int, torch.Tensor] = {
            call: torch.zeros((num_slots,) + tuple(s.shape), dtype=getattr(torch, s.dtype), device=device)
            for call, s in specs.items()
        }

    def of_call(self, call: int) -> Optional[torch.Tensor]:
        return self.pools.get(call)

    def reset_slot(self, slot: int) -> None:
        for p in self.pools.values():
            p[slot].zero_()

    def nbytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools.values())
