"""The device side of the cache: pools of pages per group of layers, and state slots.

Layers (runs of the schedule that own a cache) are grouped by what their mixers ask for:
paged keys and values with the same window, number of KV heads and head size share a group,
hence a page pool, a free list and block tables (``return_b200/cache/manager.py``).  The pool of
a group is one tensor ``[layers, 2, num_pages, Hkv, page_size, D]`` in the activation dtype
(index 0 of the second axis: keys, 1: values), so one page id addresses a slab in every layer of
the group, as in the reference (rollout/cache.py:19-24), and one (page, kv head) tile is
contiguous.  A mixer that asks for state of fixed size gets ``[max_reside + 1, *shape]``, one row per
request slot and a last one that belongs to no request (the padding rows of a captured decode step
point at it) (after rollout/cache.py:340-360).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import BuildEnv, KVCacheNeed, KVView, LayerContext, StateNeed
from .manager import CacheManager, GroupSpec


class CacheStorage:
    def __init__(self, needs: List[object], page_size: int, num_pages: int, max_reside: int, env: BuildEnv,
                 longest_append: Optional[int] = None):
        """``num_pages``: pages of a group that keeps every key (the pool's capacity in tokens / page size).
        A group that keeps a window gets only what ``max_reside`` requests can hold of it at a time: the
        window plus the longest run of tokens one step may append (``longest_append``; None: unknown, the
        group then gets ``num_pages`` too), in pages, plus one for the ragged ends."""
        self.env = env
        self.page_size = page_size
        self.max_reside = max_reside
        signature_to_group: Dict[Tuple, int] = {}
        self.group_specs: List[GroupSpec] = []
        self._group_layers: List[int] = []
        self._group_shape: List[Tuple[int, int]] = []
        self.entry_place: Dict[int, Tuple[int, int]] = {}      # schedule index -> (group, layer in group)
        self._state_needs: Dict[int, StateNeed] = {}
        for index, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, KVCacheNeed):
                sig = (need.window, need.num_kv_heads, need.head_dim)
                if sig not in signature_to_group:
                    signature_to_group[sig] = len(self.group_specs)
                    name = "full" if need.window is None else f"window{need.window}"
                    pages = num_pages
                    if need.window is not None and longest_append is not None:
                        per_request = (need.window + longest_append + page_size - 1) // page_size + 1
                        pages = max(1, min(num_pages, max_reside * per_request))
                    self.group_specs.append(GroupSpec(f"{name}_h{need.num_kv_heads}_d{need.head_dim}",
                                                      page_size, pages, need.window))
                    self._group_layers.append(0)
                    self._group_shape.append((need.num_kv_heads, need.head_dim))
                g = signature_to_group[sig]
                self.entry_place[index] = (g, self._group_layers[g])
                self._group_layers[g] += 1
            elif isinstance(need, StateNeed):
                self._state_needs[index] = need
            else:
                raise TypeError(f"schedule entry {index}: unknown cache need {need!r}")
        if not self.group_specs:
            # a model without paged layers still counts tokens per request
            self.group_specs.append(GroupSpec("none", page_size, num_pages, None))
            self._group_layers.append(0)
            self._group_shape.append((0, 0))
        self.pools: List[Optional[torch.Tensor]] = []
        self._layer_views: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]] = {}
        self.states: Dict[int, torch.Tensor] = {}

    def make_manager(self) -> CacheManager:
        manager = CacheManager(self.group_specs, self.max_reside)
        manager.on_slot_taken.append(self.reset_slot)
        manager.truncatable = not self._state_needs
        return manager

    def allocate(self) -> None:
        dev, dt = self.env.device, self.env.act_dtype
        self.pools = []
        self._layer_views = {}
        for spec, layers, (hkv, d) in zip(self.group_specs, self._group_layers, self._group_shape):
            if layers == 0:
                self.pools.append(None)
                continue
            self.pools.append(torch.zeros((layers, 2, spec.num_pages, hkv, spec.page_size, d), dtype=dt, device=dev))
        self.states = {i: torch.zeros((self.max_reside + 1,) + tuple(n.shape), dtype=n.dtype, device=dev)
                       for i, n in self._state_needs.items()}

    def bytes_per_token(self) -> int:
        total = 0
        for layers, (hkv, d) in zip(self._group_layers, self._group_shape):
            total += layers * 2 * hkv * d * torch.empty((), dtype=self.env.act_dtype).element_size()
        return total

    def poison(self) -> None:
        """Fills every page with NaN, so that a read of a slot nobody wrote shows in the logits."""
        for p in self.pools:
            if p is not None:
                p.fill_(float("nan"))

    def reset_slot(self, slot: int) -> None:
        """A request that takes a slot starts from zero state."""
        for t in self.states.values():
            t[slot].zero_()                  # in stream order: after the last step of whoever held the slot before

    def layer_context(self, owner_index: int, batch, write: bool) -> LayerContext:
        ctx = LayerContext(batch=batch, write_cache=write)
        place = self.entry_place.get(owner_index)
        if place is not None:
            g, layer = place
            views = self._layer_views.get(place)
            if views is None:                # the views of a layer's keys and values are made once
                pool = self.pools[g]
                views = self._layer_views[place] = (pool[layer, 0], pool[layer, 1])
            ctx.kv = KVView(k=views[0], v=views[1], block_table=batch.block_tables[g],
                            page_size=self.group_specs[g].page_size)
        if owner_index in self.states:
            ctx.state = self.states[owner_index]
        return ctx
