"""Device memory behind the cache manager's ids.

For each group one tensor ``[caches, 2, pages, kv heads, page_size, head_dim]``
(keys at index 0, values at index 1; ``[caches, 1, ...]`` for a group that keeps keys
only) in the run's dtype: a page id is valid for every cache of the group.  In a group whose values have another
size than its keys, the values lie in a tensor of their own, ``[caches, 1, pages, kv heads, page_size, value_dim]``.
For each state cache one tensor
``[request slots + 1, *shape]``, zeroed for a slot when a request takes it.  The last
slot belongs to no request: the rows that pad a captured decode batch name it, so a
mixer that updates ``state[state_slots]`` with device operations alone harms nobody.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .manager import CacheManager


@dataclass
class KVCacheView:
    """What an attention-like mixer gets for one run of its layer."""

    k: torch.Tensor          # [pages, kv heads, page_size, head_dim]
    v: Optional[torch.Tensor]   # None in a group that keeps keys only
    group: int               # index into StepContext.kv_groups
    page_size: int
    writes: bool             # False: this run only reads a cache another run wrote


@dataclass
class StateView:
    """What a mixer with fixed-size state gets: ``state[slot]`` belongs to the
    request whose slot is ``slot`` (StepContext.state_slots)."""

    state: torch.Tensor      # [request slots + 1, *shape]; the last slot is the padding rows' scratch
    writes: bool = True


class CacheStorage:
    def __init__(self, manager: CacheManager, state_needs: dict, dtype: torch.dtype, device):
        self.manager = manager
        self.kv: list[torch.Tensor] = []
        self.kv_values: list[Optional[torch.Tensor]] = []     # per group: the values' own tensor, where they need one
        for g in manager.groups:
            vd = getattr(g.key, "value_dim", None)
            apart = g.key.values and vd is not None and vd != g.key.head_dim
            shape = (len(g.caches), 2 if g.key.values and not apart else 1, g.pool.num_pages, g.key.num_kv_heads,
                     manager.page_size, g.key.head_dim)
            self.kv.append(torch.zeros(shape, dtype=dtype, device=device))
            self.kv_values.append(torch.zeros((*shape[:1], 1, *shape[2:5], vd), dtype=dtype, device=device) if apart else None)
        self.state: dict[str, torch.Tensor] = {
            name: torch.zeros((manager.max_requests + 1, *need.shape), dtype=need.dtype, device=device)
            for name, need in state_needs.items()
        }

    def kv_view(self, cache_name: str, writes: bool) -> KVCacheView:
        gi, ci = self.manager.group_of[cache_name]
        t, tv = self.kv[gi], self.kv_values[gi]
        v = tv[ci, 0] if tv is not None else (t[ci, 1] if t.shape[1] > 1 else None)
        return KVCacheView(k=t[ci, 0], v=v, group=gi, page_size=self.manager.page_size, writes=writes)

    def state_view(self, cache_name: str, writes: bool = True) -> StateView:
        return StateView(self.state[cache_name], writes)

    def reset_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def poison(self, group: int, pages, value: float = 3.0e4) -> None:
        """Overwrites the keys of ``pages`` with ``value`` and their values with ``-value`` in every
        cache of the group (debugging: what a freed page held must never reach a result)."""
        idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.kv[group].device)
        self.kv[group][:, 0].index_fill_(1, idx, value)
        if self.kv[group].shape[1] > 1:
            self.kv[group][:, 1].index_fill_(1, idx, -value)
        if self.kv_values[group] is not None:
            self.kv_values[group][:, 0].index_fill_(1, idx, -value)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.kv_values if t is not None) + \
            sum(t.numel() * t.element_size() for t in self.state.values())
