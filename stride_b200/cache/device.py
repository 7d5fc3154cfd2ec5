"""Device memory of the cache: pages of keys and values for every cache slot,
and per-request state slots.

Cache slots whose mixers ask for the same page geometry and the same window
form a group: one pool of page ids in the cache manager, one tensor here of
shape [slots_in_group, 2 (key, value), num_pages, kv_heads, page_size, head_dim].
Within a page the layout is [kv_head, slot, head_dim], so the keys of one head
in one page are contiguous. The reference keeps [page, slot, kv_head, head_dim]
per layer and one id space for all layers (python/stride_worker/cache.py:44-56).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache."""
    group: int                          # index into ctx.block_table / ctx.slot_mapping
    k_pages: Optional[torch.Tensor]     # [num_pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor]
    page_size: int
    writes: bool                        # False: this run reads what another run wrote
    state: Optional[torch.Tensor]       # [num_state_slots, *shape] or None


@dataclass(frozen=True)
class GroupLayout:
    num_kv_heads: int
    head_dim: int
    window: int                         # 0: every key is kept
    slots: tuple                        # cache slots in this group

    def bytes_per_page(self, page_size: int, itemsize: int) -> int:
        return 2 * len(self.slots) * self.num_kv_heads * page_size * self.head_dim * itemsize


def plan_groups(cache_requests) -> list[GroupLayout]:
    """Groups cache slots by (kv_heads, head_dim, window). A model without any
    paged mixer still gets one (empty) group so that the block-table plumbing is
    uniform."""
    by_key: dict = {}
    for slot, (req, _state) in enumerate(cache_requests):
        if req is None:
            continue
        key = (req.num_kv_heads, req.head_dim, 0 if req.window is None else int(req.window))
        by_key.setdefault(key, []).append(slot)
    groups = [GroupLayout(k[0], k[1], k[2], tuple(v)) for k, v in by_key.items()]
    return groups or [GroupLayout(0, 0, 0, ())]


class DeviceCache:
    def __init__(self, model, page_size: int, num_pages: int, num_state_slots: int, dtype: torch.dtype, device):
        self.page_size, self.num_pages, self.num_state_slots = page_size, num_pages, num_state_slots
        self.dtype, self.device = dtype, torch.device(device)
        requests = model.cache_requests()
        self.groups = plan_groups(requests)
        self.pages = []
        for g in self.groups:
            shape = (len(g.slots), 2, num_pages, g.num_kv_heads, page_size, g.head_dim)
            self.pages.append(torch.zeros(shape, dtype=dtype, device=self.device) if g.slots else None)
        self.states = {}
        for slot, (_req, state) in enumerate(requests):
            if state is not None:
                self.states[slot] = torch.zeros((num_state_slots, *state.shape), dtype=state.dtype, device=self.device)
        slot_group = {s: gi for gi, g in enumerate(self.groups) for s in g.slots}
        caches = []
        for entry in model.schedule:
            gi = slot_group.get(entry.cache)
            if gi is None:
                caches.append(LayerCache(0, None, None, page_size, entry.writes_cache, self.states.get(entry.cache)))
                continue
            index = self.groups[gi].slots.index(entry.cache)
            caches.append(LayerCache(gi, self.pages[gi][index, 0], self.pages[gi][index, 1], page_size,
                                     entry.writes_cache, self.states.get(entry.cache)))
        model.caches = caches

    def group_configs(self) -> list[tuple]:
        """(num_pages, window) per group, for the cache manager."""
        return [(self.num_pages, g.window) for g in self.groups]

    def bytes_per_page(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_page(self.page_size, item) for g in self.groups)

    def total_bytes(self) -> int:
        total = sum(p.numel() * p.element_size() for p in self.pages if p is not None)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())

    def zero_(self) -> None:
        for p in self.pages:
            if p is not None:
                p.zero_()
        for s in self.states.values():
            s.zero_()
