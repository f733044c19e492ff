"""Device memory of the cache: pages per layer group, and the rows of fixed-size per-request
state, laid out from what the model's mixers say they need."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import KVNeed, PagedNeed, StateNeed
from .manager import CacheManager, KVGroupSpec


@dataclass
class LayerCache:
    """What one execution of a mixer sees of the cache."""
    layer: int
    group: int = -1                     # layer group of a paged layer
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)   # name -> [page, heads, page_tokens, width]
    state: Optional[torch.Tensor] = None  # [max_requests + 1, *shape] of a stateful mixer
    writes: bool = True

    @property
    def k(self) -> Optional[torch.Tensor]:
        return self.tensors.get("k")

    @property
    def v(self) -> Optional[torch.Tensor]:
        return self.tensors.get("v")


class CacheStorage:
    """Groups the model's cache layers by need, creates the manager and the tensors.

    Paged layout per group and named tensor: [layer_in_group, page, heads, page_tokens, width]:
    one page id is valid in every layer and every tensor of the group, and what one (page,
    head) holds is a contiguous [page_tokens, width] tile.  The usual need is a key and a
    value tensor of equal geometry (``KVNeed``); a ``PagedNeed`` lists any other set.  The
    reference keeps one K pool and one V pool per layer, [num_blocks, block_size * kv_heads *
    head_dim] (infMain/source/base/block_allocator.cpp:46-49)."""

    def __init__(self, needs: Sequence[object], page_tokens: int, num_pages, max_requests: int,
                 dtype: torch.dtype, device, lifo: bool = False, poison: bool = False):
        self.page_tokens, self.dtype, self.device = int(page_tokens), dtype, device
        keys: List[tuple] = []
        members: Dict[tuple, List[int]] = {}
        self._layer_group: Dict[int, int] = {}
        self._layer_index: Dict[int, int] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.max_requests = int(max_requests)
        for layer, need in enumerate(needs):
            if isinstance(need, (KVNeed, PagedNeed)):
                key = (tuple(need.tensors), need.window)
                if not key[0]:
                    raise TypeError(f"cache layer {layer}: a paged need lists at least one tensor")
                if len({t.name for t in key[0]}) != len(key[0]):
                    raise TypeError(f"cache layer {layer}: two cache tensors share a name")
                if key not in members:
                    members[key] = []
                    keys.append(key)
                self._layer_group[layer] = keys.index(key)
                self._layer_index[layer] = len(members[key])
                members[key].append(layer)
            elif isinstance(need, StateNeed):
                # one row per request slot and one more, which the padding rows of captured
                # decode steps point at
                self.state[layer] = torch.zeros((self.max_requests + 1,) + tuple(need.shape), dtype=need.dtype,
                                                device=device)
            elif need is not None:
                raise TypeError(f"cache layer {layer}: unknown need {need!r}")
        groups = [KVGroupSpec(tuple(members[k]), k[0][0].heads, k[0][0].width, k[1], tensors=k[0]) for k in keys]
        self.manager = CacheManager(groups, page_tokens, num_pages if groups else [], max_requests,
                                    lifo=lifo)
        self.paged: List[Dict[str, torch.Tensor]] = []
        for g, spec in enumerate(groups):
            n = self.manager.pools[g].num_pages
            held = {}
            for t in spec.tensors:
                x = torch.empty((len(spec.layers), n, t.heads, self.page_tokens, t.width), dtype=dtype, device=device)
                if poison:
                    x.fill_(float("nan"))
                held[t.name] = x
            self.paged.append(held)

    @property
    def groups(self):
        return self.manager.groups

    @property
    def state_pad_slot(self) -> int:
        """The row of the state tensors that belongs to no request."""
        return self.max_requests

    def bytes_per_token(self) -> int:
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * sum(t.heads * t.width for t in g.tensors) * size for g in self.groups)

    def zero_state(self, slots) -> None:
        """Zeroes the state rows of these request slots in every stateful layer (the step
        function calls it for requests whose first tokens are about to run)."""
        if not self.state or len(slots) == 0:
            return
        idx = torch.as_tensor(list(slots), dtype=torch.long).to(self.device)
        for t in self.state.values():
            t.index_fill_(0, idx, 0)

    def layer(self, cache_layer: int, writes: bool = True) -> LayerCache:
        if cache_layer in self._layer_group:
            g, i = self._layer_group[cache_layer], self._layer_index[cache_layer]
            return LayerCache(layer=cache_layer, group=g, tensors={n: t[i] for n, t in self.paged[g].items()},
                              writes=writes)
        if cache_layer in self.state:
            return LayerCache(layer=cache_layer, state=self.state[cache_layer], writes=writes)
        return LayerCache(layer=cache_layer, writes=writes)
