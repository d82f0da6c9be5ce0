"""Device side of the cache: per layer the K and V page pools, or the state
tensor, laid out for the page and slot numbers of ``PageTable``.

The K pool of a layer is [pages, kv_heads, page_size, head_dim], its V pool
[pages, kv_heads, page_size, v_head_dim] (as wide as the keys unless the mixer
says otherwise): the ``page_size x width`` slab of one (page, head) is
contiguous.  Pages are
never cleared: what a request may read is decided by its length, not by the
pages' content.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..parts.base import CacheNeed, LayerCache
from .manager import GroupSpec, PageTable


def group_layers(needs: List[CacheNeed]) -> Tuple[List[Tuple[int, int, int, int, bool]], List[int]]:
    """Group keys (kv_heads, head_dim, window, value width, values inside the keys) in order of first use,
    and for every layer the index of its group (-1: the layer holds no pages)."""
    keys: List[Tuple[int, int, int, int, bool]] = []
    of_layer: List[int] = []
    for need in needs:
        if need.kind == "multi":
            # the page-holding parts of a mixer made of mixers join the groups like layers of their own;
            # the need itself holds no pages
            for part in need.flat():
                if part.kind == "kv":
                    key = (part.kv_heads, part.head_dim, part.window, part.value_dim, part.values_in_keys)
                    if key not in keys:
                        keys.append(key)
            of_layer.append(-1)
            continue
        if need.kind != "kv":
            of_layer.append(-1)
            continue
        key = (need.kv_heads, need.head_dim, need.window, need.value_dim, need.values_in_keys)
        if key not in keys:
            keys.append(key)
        of_layer.append(keys.index(key))
    return keys, of_layer


def bytes_per_page(needs: List[CacheNeed], page_size: int, elem_size: int) -> List[int]:
    """Per group, the bytes one page number costs across the group's layers."""
    keys, _ = group_layers(needs)
    flat = [f for need in needs for f in need.flat()]
    _, of_layer = group_layers(flat)
    out = [0] * len(keys)
    for need, g in zip(flat, of_layer):
        if g >= 0:
            width = need.head_dim + (0 if need.values_in_keys else need.value_dim)
            out[g] += need.kv_heads * page_size * width * elem_size
    return out


class CachePools:
    def __init__(self, needs: List[CacheNeed], pages_per_group: List[int], page_size: int,
                 max_requests: int, dtype: torch.dtype, device):
        self.needs = needs
        keys, self.group_of_layer = group_layers(needs)
        if len(pages_per_group) != len(keys):
            raise ValueError("one page count per layer group is needed")
        self.groups = [GroupSpec(pages_per_group[g], page_size, keys[g][2]) for g in range(len(keys))]
        # A model none of whose layers holds pages (recurrent layers only) still has the table count its
        # requests' tokens and hand out state slots: one group of page numbers that stand for no storage
        # and do not run out.
        self.table = PageTable(self.groups, max_requests) if keys else PageTable(
            [GroupSpec(1 << 20, page_size, 0)], max_requests)
        self.page_size = page_size
        def storage(need: CacheNeed) -> LayerCache:
            if need.kind == "multi":
                return LayerCache(need, -1, parts=tuple(storage(p) for p in need.parts))
            if need.kind == "kv":
                g = keys.index((need.kv_heads, need.head_dim, need.window, need.value_dim, need.values_in_keys))
                k_shape = (pages_per_group[g], need.kv_heads, page_size, need.head_dim)
                v_shape = (pages_per_group[g], need.kv_heads, page_size, need.value_dim)
                # zeros, not uninitialised memory: rows that a tile loads but masks must be finite
                k_pool = torch.zeros(k_shape, dtype=dtype, device=device)
                v_pool = k_pool if need.values_in_keys else torch.zeros(v_shape, dtype=dtype, device=device)
                return LayerCache(need, g, k_pool, v_pool, page_size)
            if need.kind == "state":
                st = torch.zeros((max_requests, *need.state_shape), dtype=need.state_dtype,
                                 device=device)
                return LayerCache(need, -1, state=st)
            return LayerCache(need)

        self.layers: List[LayerCache] = [storage(need) for need in needs]

    def nbytes(self) -> int:
        def size(lc: LayerCache) -> int:
            own = sum(t.numel() * t.element_size() for t in (lc.k, lc.v if lc.v is not lc.k else None, lc.state)
                      if t is not None)
            return own + sum(size(p) for p in lc.parts)

        return sum(size(lc) for lc in self.layers)
