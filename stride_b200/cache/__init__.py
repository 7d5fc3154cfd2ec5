"""The cache: host bookkeeping (pages, block tables, prefix index, state slots;
C++, ``csrc/runtime``) and the device tensors that the pages name."""

from ..csrc.build import load_runtime
from .device import DeviceCache, GroupLayout, LayerCache, plan_groups


def runtime():
    """The compiled host runtime module (built on first use)."""
    return load_runtime()


def CacheManager(page_size: int, groups, num_state_slots: int, prefix_caching: bool = True):
    """groups: list of (num_pages, window) with window 0 for 'keeps every key'."""
    return load_runtime().CacheManager(page_size, [(int(n), int(w)) for n, w in groups], num_state_slots, prefix_caching)


__all__ = ["CacheManager", "DeviceCache", "GroupLayout", "LayerCache", "plan_groups", "runtime"]
