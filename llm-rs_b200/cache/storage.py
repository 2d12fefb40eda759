"""Device memory of the cache: pages of keys and values per group, state per slot.

One group's pages are one tensor ``[entries, n_pages, n_kv_heads, page_size * sum(widths)]`` in the
activation type, ``widths`` being the group's planes (``CacheNeed.plane_widths``): the rows of one
(page, head, plane) are ``page_size * width`` contiguous elements and a head's planes follow one
another, so a kernel fetches a tile with one straight copy. For the usual two planes of equal width
(keys and values) that is ``[entries, n_pages, n_kv_heads, 2, page_size, head_dim]``, which is the
view attention gets. Fixed-size state is ``[n_slots, *shape]`` float32 per run-order entry
that asked for it, zeroed when a request takes the slot.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.spec import CacheNeed, RunStep, StateNeed
from .manager import GroupSpec


def plan_groups(needs: Sequence[Tuple[Optional[CacheNeed], Optional[StateNeed]]], run_order: Sequence[RunStep],
                n_pages: int) -> Tuple[List[GroupSpec], List[Optional[int]], List[Optional[int]]]:
    """Sort run-order entries into groups by need.

    Returns (groups, entry_group, entry_index): for entry s, ``entry_group[s]`` is its
    group and ``entry_index[s]`` its place in the group's tensor; an entry that reads
    another entry's cache gets that entry's pair; an entry without pages gets None.
    """
    groups: List[GroupSpec] = []
    by_key: Dict[tuple, int] = {}
    entry_group: List[Optional[int]] = [None] * len(run_order)
    entry_index: List[Optional[int]] = [None] * len(run_order)
    for s, (need, _) in enumerate(needs):
        if run_order[s].cache_of is not None or need is None:
            continue
        key = need.group_key()
        if key not in by_key:
            by_key[key] = len(groups)
            groups.append(GroupSpec(need=need, entries=[], n_pages=n_pages))
        g = by_key[key]
        entry_group[s], entry_index[s] = g, len(groups[g].entries)
        groups[g].entries.append(s)
    for s, step in enumerate(run_order):
        if step.cache_of is not None:
            entry_group[s], entry_index[s] = entry_group[step.cache_of], entry_index[step.cache_of]
    return groups, entry_group, entry_index


class LayerCache:
    """What a mixer sees of the cache for one run-order entry in one step."""
    __slots__ = ("kv", "planes", "block_table", "page_size", "owns", "state", "group")

    def __init__(self, kv, planes, block_table, page_size, owns, state, group):
        self.kv = kv                    # [n_pages, n_kv_heads, 2, page_size, head_dim] (two equal planes) or None
        self.planes = planes            # per plane: [n_pages, n_kv_heads, page_size, width] (a view), or None
        self.block_table = block_table  # int32 [requests of the step, pages] or None
        self.page_size = page_size
        self.owns = owns                # False: reads another entry's keys and values, writes none
        self.state = state              # name -> [n_slots, *shape] float32
        self.group = group


class CacheStorage:
    def __init__(self, needs, run_order: Sequence[RunStep], page_size: int, n_pages: int, n_slots: int,
                 dtype: torch.dtype, device):
        self.page_size, self.n_slots, self.dtype, self.device = page_size, n_slots, dtype, device
        self.run_order = list(run_order)
        self.groups, self.entry_group, self.entry_index = plan_groups(needs, run_order, n_pages)
        self._view_cache: Dict[tuple, tuple] = {}
        self.kv: List[torch.Tensor] = []      # per group: [entries, pages, heads, page_size * sum(widths)]
        for g in self.groups:
            shape = (len(g.entries), g.n_pages, g.need.n_kv_heads, page_size * sum(g.need.plane_widths))
            self.kv.append(torch.zeros(shape, dtype=dtype, device=device))
        self.state: List[Dict[str, torch.Tensor]] = []
        for s, (_, st) in enumerate(needs):
            tensors = {}
            if st is not None and self.run_order[s].cache_of is None:
                for name, shape in st.tensors.items():
                    tensors[name] = torch.zeros((n_slots, *shape), dtype=torch.float32, device=device)
            self.state.append(tensors)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + sum(
            t.numel() * 4 for d in self.state for t in d.values())

    def reset_slot(self, slot: int) -> None:
        """Zero the fixed-size state of a slot (a new request takes it)."""
        for tensors in self.state:
            for t in tensors.values():
                t[slot].zero_()

    def snapshot_state(self, slots: Sequence[int]):
        """Copies of the fixed-size state that the given slots hold (for ``restore_state``)."""
        if not any(self.state):
            return []
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        return [(t, idx, t.index_select(0, idx)) for tensors in self.state for t in tensors.values()]

    @staticmethod
    def restore_state(saved) -> None:
        for t, idx, copy in saved:
            t.index_copy_(0, idx, copy)

    def layer_cache(self, s: int, block_tables: Sequence[Optional[torch.Tensor]]) -> LayerCache:
        g, i = self.entry_group[s], self.entry_index[s]
        src = self.run_order[s].cache_of
        state = self.state[s if src is None else src]
        if g is None:
            return LayerCache(None, None, None, self.page_size, src is None, state, None)
        kv, planes = self._views(g, i)
        return LayerCache(kv, planes, block_tables[g], self.page_size, src is None, state, g)

    def _views(self, g: int, i: int):
        """The views of entry ``i`` of group ``g`` that a mixer gets (made once: they do not change)."""
        views = self._view_cache.get((g, i))
        if views is None:
            flat = self.kv[g][i]                                    # [pages, heads, page_size * sum(widths)]
            widths = self.groups[g].need.plane_widths
            planes, at = [], 0
            for w in widths:
                planes.append(flat[:, :, at:at + self.page_size * w].unflatten(2, (self.page_size, w)))
                at += self.page_size * w
            kv = None
            if len(widths) == 2 and widths[0] == widths[1]:
                kv = flat.view(flat.size(0), flat.size(1), 2, self.page_size, widths[0])
            views = self._view_cache[(g, i)] = (kv, planes)
        return views
