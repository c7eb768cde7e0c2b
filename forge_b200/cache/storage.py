"""Device storage behind the cache manager, laid out from the model's schedule of layer runs.

Every run of a layer's mixer states what it needs (``cache_spec``): keys/values in pages, fixed-size
state, or nothing.  Runs with equal key/value needs share a group (one page pool, one block table per
request); each such run owns a tensor [num_pages, 2, kv_heads, page_size, head_dim] with a page's keys
and values adjacent.  A state-keeping run owns a tensor [max_requests, *shape] addressed by request slot.
A run whose layer says ``cache_from`` gets a read-only view of an earlier run's storage and allocates
nothing.  ("Layer" below means one position of the schedule.)
"""
from dataclasses import dataclass
from typing import Optional

import torch

from ..parts.base import KVCacheSpec, StateSpec
from .manager import CacheManager, GroupSpec
from .pages import CacheError


@dataclass
class LayerCache:
    """What a mixer gets: its group's name (to find block table and slot mapping in the step's batch), its
    storage, and whether it may write."""
    group: Optional[str]
    page_size: int
    kv: Optional[torch.Tensor] = None          # [num_pages, 2, NKV, page_size, HD]
    state: Optional[torch.Tensor] = None       # [max_requests, *shape]
    writable: bool = True


def group_name(spec: KVCacheSpec):
    w = "full" if spec.window is None else f"win{spec.window}"
    return f"kv{spec.num_kv_heads}x{spec.head_dim}_{w}"


def plan_groups(cache_specs, cache_from):
    """cache_specs: per layer KVCacheSpec | StateSpec | None.  Returns ({group name: KVCacheSpec},
    per-layer group name or None)."""
    groups, layer_group = {}, []
    for i, spec in enumerate(cache_specs):
        src = cache_from[i]
        if src is not None:
            s2 = cache_specs[src]
            if cache_from[src] is not None:
                raise CacheError(f"layer {i} reads the cache of layer {src}, which has none of its own")
            if isinstance(spec, KVCacheSpec) and isinstance(s2, KVCacheSpec) and \
                    (spec.num_kv_heads, spec.head_dim) != (s2.num_kv_heads, s2.head_dim):
                raise CacheError(f"layer {i} cannot read the cache of layer {src}: shapes differ")
            spec = s2
        if isinstance(spec, KVCacheSpec):
            name = group_name(spec)
            groups[name] = spec
            layer_group.append(name)
        else:
            layer_group.append(None)
    return groups, layer_group


def bytes_per_page(cache_specs, cache_from, page_size, dtype):
    """{group: bytes one page takes over all layers of the group that own storage}."""
    groups, layer_group = plan_groups(cache_specs, cache_from)
    el = torch.empty((), dtype=dtype).element_size()
    out = {g: 0 for g in groups}
    for i, spec in enumerate(cache_specs):
        if cache_from[i] is None and isinstance(spec, KVCacheSpec):
            out[layer_group[i]] += 2 * spec.num_kv_heads * page_size * spec.head_dim * el
    return out


class CacheStorage:
    def __init__(self, cache_specs, cache_from, page_size, pages_per_group, max_requests, dtype, device):
        """pages_per_group: int (same for every group) or {group: int}."""
        groups, self.layer_group = plan_groups(cache_specs, cache_from)
        if isinstance(pages_per_group, int):
            pages_per_group = {g: pages_per_group for g in groups}
        self.manager = CacheManager([GroupSpec(g, pages_per_group[g], s.window) for g, s in groups.items()],
                                    page_size, max_requests)
        self.page_size, self.max_requests, self.dtype, self.device = page_size, max_requests, dtype, device
        self.layers = []
        self._state_tensors = []
        self._guarded = []              # (what, whole allocation): one page (or row) of canary words before and after
        for i, spec in enumerate(cache_specs):
            if cache_from[i] is not None:
                self.layers.append(None)       # filled below
                continue
            if isinstance(spec, KVCacheSpec):
                kv = self._guarded_zeros(f"keys/values of run {i}", (pages_per_group[self.layer_group[i]], 2, spec.num_kv_heads,
                                                                     page_size, spec.head_dim), dtype)
                self.layers.append(LayerCache(self.layer_group[i], page_size, kv=kv))
            elif isinstance(spec, StateSpec):
                st = self._guarded_zeros(f"state of run {i}", (max_requests, *spec.shape), spec.dtype)
                self._state_tensors.append(st)
                self.layers.append(LayerCache(None, page_size, state=st))
            elif spec is None:
                self.layers.append(LayerCache(None, page_size))
            else:
                raise CacheError(f"layer {i}: unknown cache spec {spec!r}")
        for i, src in enumerate(cache_from):
            if src is not None:
                s = self.layers[src]
                self.layers[i] = LayerCache(s.group, page_size, kv=s.kv, state=s.state, writable=False)

    # Canary words: every cache tensor is allocated with one more page (or state row) in front and one behind, filled
    # with a fixed bit pattern that nothing ever writes.  A kernel that follows a page id of -1 or num_pages (or a slot
    # past the pool) writes there instead of into a neighbour's memory, and check_canaries() says which tensor it was.
    CANARY_BYTE = 0x5A

    def _guarded_zeros(self, what, shape, dtype):
        whole = torch.zeros((shape[0] + 2, *shape[1:]), dtype=dtype, device=self.device)
        whole[0].view(torch.uint8).fill_(self.CANARY_BYTE)
        whole[-1].view(torch.uint8).fill_(self.CANARY_BYTE)
        self._guarded.append((what, whole))
        return whole[1:-1]

    def check_canaries(self):
        """Names of the cache tensors whose guard words were overwritten (synchronises)."""
        bad = []
        for what, whole in self._guarded:
            for edge, name in ((whole[0], "before"), (whole[-1], "behind")):
                if not bool((edge.view(torch.uint8) == self.CANARY_BYTE).all()):
                    bad.append(f"{what} (the guard {name} it)")
        return bad

    def zero_state_slots(self, slots):
        """Clears the state rows of newly admitted requests."""
        if slots and self._state_tensors:
            idx = torch.tensor(slots, dtype=torch.long, device=self.device)
            for st in self._state_tensors:
                st.index_fill_(0, idx, 0)
