"""Device memory of the cache: pages for every cache slot, and per-request state slots.

A mixer says what it keeps per token (``CacheRequest.layout()``: named tensors of [heads, width]; keys and values
of one shape in the plain case). Cache slots whose mixers ask for the same layout and the same window form a
group: one pool of page ids in the cache manager, and here one tensor per name of shape
[slots_in_group, num_pages, heads, page_size, width]. Within a page the layout is [head, slot, width], so what
one head keeps in one page is contiguous. The reference keeps [page, slot, kv_head, head_dim] per layer and one id
space for all layers (python/stride_worker/cache.py:44-56).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache."""
    group: int                          # index into ctx.block_table / ctx.slot_mapping
    k_pages: Optional[torch.Tensor]     # [num_pages, kv_heads, page_size, head_dim]: the tensors named "k" and "v", if any
    v_pages: Optional[torch.Tensor]
    page_size: int
    writes: bool                        # False: this run reads what another run wrote
    state: Optional[torch.Tensor]       # [num_state_slots, *shape] or None
    tensors: dict = field(default_factory=dict)     # name -> [num_pages, heads, page_size, width], every paged tensor of the slot


@dataclass(frozen=True)
class GroupLayout:
    layout: tuple                       # of (name, heads, width): what a token keeps in this group
    window: int                         # 0: every token is kept
    slots: tuple                        # cache slots in this group

    @property
    def num_kv_heads(self) -> int:
        return self.layout[0][1] if self.layout else 0

    @property
    def head_dim(self) -> int:
        return self.layout[0][2] if self.layout else 0

    def elements_per_token(self) -> int:
        return len(self.slots) * sum(h * w for _n, h, w in self.layout)

    def bytes_per_page(self, page_size: int, itemsize: int) -> int:
        return self.elements_per_token() * page_size * itemsize


def plan_groups(cache_requests) -> list[GroupLayout]:
    """Groups cache slots by (layout, window). A model without any paged mixer still gets one (empty) group so that
    the block-table plumbing is uniform."""
    by_key: dict = {}
    for slot, (req, _state) in enumerate(cache_requests):
        if req is None:
            continue
        key = (req.layout(), 0 if req.window is None else int(req.window))
        by_key.setdefault(key, []).append(slot)
    groups = [GroupLayout(k[0], k[1], tuple(v)) for k, v in by_key.items()]
    return groups or [GroupLayout((), 0, ())]


class DeviceCache:
    def __init__(self, model, page_size: int, num_pages: int, num_state_slots: int, dtype: torch.dtype, device):
        self.page_size, self.num_pages, self.num_state_slots = page_size, num_pages, num_state_slots
        self.dtype, self.device = dtype, torch.device(device)
        requests = model.cache_requests()
        self.groups = plan_groups(requests)
        self.group_tensors = []         # per group: name -> [slots_in_group, num_pages, heads, page_size, width]
        self.pages = []                 # every paged tensor, flat (to fill, poison or count them)
        for g in self.groups:
            named = {}
            for name, heads, width in (g.layout if g.slots else ()):
                named[name] = torch.zeros((len(g.slots), num_pages, heads, page_size, width), dtype=dtype, device=self.device)
                self.pages.append(named[name])
            self.group_tensors.append(named)
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
            named = {name: t[index] for name, t in self.group_tensors[gi].items()}
            caches.append(LayerCache(gi, named.get("k"), named.get("v"), page_size, entry.writes_cache,
                                     self.states.get(entry.cache), named))
        model.caches = caches

    def group_configs(self) -> list[tuple]:
        """(num_pages, window) per group, for the cache manager."""
        return [(self.num_pages, g.window) for g in self.groups]

    def bytes_per_page(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_page(self.page_size, item) for g in self.groups)

    def total_bytes(self) -> int:
        total = sum(p.numel() * p.element_size() for p in self.pages)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())

    def zero_(self) -> None:
        for p in self.pages:
            p.zero_()
        for s in self.states.values():
            s.zero_()
