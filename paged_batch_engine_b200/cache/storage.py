"""Device memory of the cache: pages of keys and values per layer group, and the rows of
fixed-size per-request state, laid out from what the model's mixers say they need."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import KVNeed, StateNeed
from .manager import CacheManager, KVGroupSpec


@dataclass
class LayerCache:
    """What one execution of a mixer sees of the cache."""
    layer: int
    group: int = -1                     # layer group of a paged layer
    k: Optional[torch.Tensor] = None    # [page, kv_head, page_tokens, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None  # [max_requests, *shape] of a stateful mixer
    writes: bool = True


class CacheStorage:
    """Groups the model's cache layers by need, creates the manager and the tensors.

    Paged layout per group: [layer_in_group, 2 (K, V), page, kv_head, page_tokens, head_dim]:
    one page id is valid in every layer of the group, and the keys of one (page, head) are a
    contiguous [page_tokens, head_dim] tile.  The reference keeps one K pool and one V pool
    per layer, [num_blocks, block_size * kv_heads * head_dim]
    (infMain/source/base/block_allocator.cpp:46-49)."""

    def __init__(self, needs: Sequence[object], page_tokens: int, num_pages, max_requests: int,
                 dtype: torch.dtype, device, lifo: bool = False, poison: bool = False):
        self.page_tokens, self.dtype, self.device = int(page_tokens), dtype, device
        keys: List[KVNeed] = []
        members: Dict[KVNeed, List[int]] = {}
        self._layer_group: Dict[int, int] = {}
        self._layer_index: Dict[int, int] = {}
        self.state: Dict[int, torch.Tensor] = {}
        for layer, need in enumerate(needs):
            if isinstance(need, KVNeed):
                if need not in members:
                    members[need] = []
                    keys.append(need)
                self._layer_group[layer] = keys.index(need)
                self._layer_index[layer] = len(members[need])
                members[need].append(layer)
            elif isinstance(need, StateNeed):
                self.state[layer] = torch.zeros((max_requests,) + tuple(need.shape), dtype=need.dtype,
                                                device=device)
            elif need is not None:
                raise TypeError(f"cache layer {layer}: unknown need {need!r}")
        groups = [KVGroupSpec(tuple(members[k]), k.num_kv_heads, k.head_dim, k.window) for k in keys]
        self.manager = CacheManager(groups, page_tokens, num_pages if groups else [], max_requests,
                                    lifo=lifo)
        self.kv: List[torch.Tensor] = []
        for g, spec in enumerate(groups):
            n = self.manager.pools[g].num_pages
            shape = (len(spec.layers), 2, n, spec.num_kv_heads, self.page_tokens, spec.head_dim)
            t = torch.empty(shape, dtype=dtype, device=device)
            if poison:
                t.fill_(float("nan"))
            self.kv.append(t)

    @property
    def groups(self):
        return self.manager.groups

    def bytes_per_token(self) -> int:
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * 2 * g.num_kv_heads * g.head_dim * size for g in self.groups)

    def layer(self, cache_layer: int, writes: bool = True) -> LayerCache:
        if cache_layer in self._layer_group:
            g, i = self._layer_group[cache_layer], self._layer_index[cache_layer]
            return LayerCache(layer=cache_layer, group=g, k=self.kv[g][i, 0], v=self.kv[g][i, 1],
                              writes=writes)
        if cache_layer in self.state:
            return LayerCache(layer=cache_layer, state=self.state[cache_layer], writes=writes)
        return LayerCache(layer=cache_layer, writes=writes)
