"""Device storage behind the cache plan of a model.

Every schedule entry that owns a paged cache gets one tensor
``[2, pages, kv_heads, page_size, head_size]`` (keys, values; two tensors
``[pages, kv_heads, page_size, size]`` where a value head is not as large as a
key head): a page of one
key/value head is ``page_size * head_size`` contiguous elements, which is the
tile the attention kernels stream.  Pages of one group share their numbering
across the layers of the group, so one block table per request serves them all
(as the single geometry of the reference does,
``src/einf/cache/storage.py:52-85``).  Entries with a state need get
``[slots, *shape]``, zeroed when a request starts.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..parts.base import CacheView, PagedKVNeed, StateNeed, pages_of, state_of
from ..parts.model import CachePlan


class CacheStorage:
    def __init__(
        self,
        plan: CachePlan,
        pages_per_group: Sequence[int],
        page_size: int,
        num_state_slots: int,
        dtype: torch.dtype,
        device: torch.device | str,
    ) -> None:
        if len(pages_per_group) != len(plan.group_windows):
            raise ValueError("one page count per cache group is needed")
        self.plan = plan
        self.page_size = page_size
        self.pages_per_group = tuple(pages_per_group)
        self.num_state_slots = num_state_slots
        self._owned: dict[int, torch.Tensor] = {}
        self._states: dict[int, torch.Tensor] = {}
        self.views: list[CacheView] = []
        for index, entry in enumerate(plan.entries):
            if entry.owner != index:
                continue
            need, state = pages_of(entry.need), state_of(entry.need)
            if need is not None and need.value_size == 0:
                # the values are read out of the key rows: keys only
                pages = self.pages_per_group[entry.group]
                self._owned[index] = (
                    torch.zeros((pages, need.num_kv_heads, page_size, need.head_size), dtype=dtype, device=device),
                    None,
                )
            elif need is not None and need.value_size != need.head_size:
                # keys and values of different sizes: one tensor each
                pages = self.pages_per_group[entry.group]
                self._owned[index] = tuple(
                    torch.zeros((pages, need.num_kv_heads, page_size, size), dtype=dtype, device=device)
                    for size in (need.head_size, need.value_size)
                )
            elif need is not None:
                self._owned[index] = torch.zeros(
                    (2, self.pages_per_group[entry.group], need.num_kv_heads, page_size, need.head_size),
                    dtype=dtype,
                    device=device,
                )
            if state is not None:
                if num_state_slots <= 0:
                    raise ValueError("the model has per-request state but the engine has no state slots")
                self._states[index] = torch.zeros((num_state_slots, *state.shape), dtype=state.dtype, device=device)
        for index, entry in enumerate(plan.entries):
            view = CacheView(writes=False)
            if pages_of(entry.need) is not None:
                kv = self._owned[entry.owner]
                view = CacheView(group=entry.group, k=kv[0], v=kv[1], writes=entry.owner == index, page_size=page_size)
            if state_of(entry.need) is not None:
                view.state = self._states[entry.owner]
                view.writes = entry.owner == index
            self.views.append(view)

    @property
    def state_tensors(self) -> list[torch.Tensor]:
        return list(self._states.values())

    def bytes(self) -> int:
        total = 0
        for owned in list(self._owned.values()) + list(self._states.values()):
            for t in (owned if isinstance(owned, tuple) else (owned,)):
                if t is None:
                    continue
                total += t.numel() * t.element_size()
        return total
