"""Device memory behind the cache manager's page ids and state slots.

The reference keeps one pool ``[L, 2, num_blocks, block_size, n_kv, d]`` (csrc/executor/kv_cache.cpp:9-25).
Here every cache group has a pool ``[runs, pages, 2, n_kv, page_size, d]``: the keys (or values) of one
page and one kv head are ``page_size * d`` contiguous elements, which is the tile an attention kernel
loads.  Per-request state of fixed size lives in ``[slots, *shape]`` tensors, one per run that asks for it.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..parts.spec import StateNeed
from .manager import CacheGroupSpec

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def page_bytes(group: CacheGroupSpec, page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id stands for: keys and values of every run of the group."""
    width = torch.empty((), dtype=dtype).element_size()
    return len(group.runs) * 2 * group.num_kv_heads * page_size * group.head_dim * width


class CacheStorage:
    def __init__(self, groups: Sequence[CacheGroupSpec], page_size: int, num_pages: Sequence[int],
                 state_needs: Dict[int, StateNeed], max_requests: int, dtype: torch.dtype, device) -> None:
        self.page_size = page_size
        self.dtype = dtype
        self.pools: List[torch.Tensor] = []
        self.run_cache: Dict[int, torch.Tensor] = {}
        self.run_group: Dict[int, int] = {}
        for g, (spec, pages) in enumerate(zip(groups, num_pages)):
            pool = torch.zeros((len(spec.runs), pages, 2, spec.num_kv_heads, page_size, spec.head_dim),
                               dtype=dtype, device=device)
            self.pools.append(pool)
            for i, run in enumerate(spec.runs):
                self.run_cache[run] = pool[i]
                self.run_group[run] = g
        self.state: Dict[int, torch.Tensor] = {}
        for run, need in state_needs.items():
            if need.dtype not in _STATE_DTYPES:
                raise ValueError(f"state dtype {need.dtype!r} is not one of {sorted(_STATE_DTYPES)}")
            self.state[run] = torch.zeros((max_requests, *need.shape), dtype=_STATE_DTYPES[need.dtype], device=device)

    def zero_slots(self, slots: Sequence[int]) -> None:
        """A request that has just been admitted starts from zero state."""
        if not slots or not self.state:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=next(iter(self.state.values())).device)
        for t in self.state.values():
            t.index_fill_(0, idx, 0)
