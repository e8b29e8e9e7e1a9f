"""Device memory behind the cache manager.

One tensor per page group, ``[stops, *need.layout(pages, page_size)]``; for
keys and values that is ``[stops, 2 (K,V), pages, kv_heads, page_size,
head_dim]``: a page of one KV head is ``page_size * head_dim`` contiguous
elements, which is the tile attention kernels stream.  (The reference's pool is
``[2, layers, pages, page_size, kv_heads, head_dim]``,
python/freetoken/kvcache/mha_pool.py:50-58.)  Page 0 is the sink that unused
block-table entries point at.  State groups are ``[stops, slots + 1, *shape]``
with the last row as the sink for padded rows
(cf. python/freetoken/kvcache/linear_state_pool.py:32-78).
"""

from __future__ import annotations

from typing import List, Sequence

import torch

from .manager import CacheManager

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    def __init__(self, manager: CacheManager, kv_dtype: torch.dtype, device):
        self.manager = manager
        self.device = torch.device(device)
        self.kv_dtype = kv_dtype
        self.paged: List[torch.Tensor] = []
        for g in manager.paged_groups:
            pages = g.pool.first_page + g.pool.num_pages
            dtype = kv_dtype if g.need.storage_dtype is None else _STATE_DTYPES[g.need.storage_dtype]
            self.paged.append(torch.zeros((len(g.stops),) + tuple(g.need.layout(pages, manager.page_size)),
                                          dtype=dtype, device=self.device))
        self.state: List[torch.Tensor] = []
        for g in manager.state_groups:
            self.state.append(torch.zeros(
                (len(g.stops), manager.max_slots + 1) + tuple(g.need.shape),
                dtype=_STATE_DTYPES[g.need.dtype], device=self.device))

    def kv_of_stop(self, stop: int) -> torch.Tensor:
        """The pages of one cache-owning stop in its need's layout (keys and
        values: ``[2, pages, kv_heads, page_size, head_dim]``)."""
        g, i = self.manager.paged_index[stop]
        return self.paged[g][i]

    def state_of_stop(self, stop: int) -> torch.Tensor:
        """``[slots + 1, *shape]`` of one cache-owning stop."""
        g, i = self.manager.state_index[stop]
        return self.state[g][i]

    def clear_state(self, slots: Sequence[int]) -> None:
        """Zero the state rows of newly admitted request slots."""
        if not slots or not self.state:
            return
        index = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        for t in self.state:
            t.index_fill_(1, index, 0)

    def poison(self, group: int, pages: Sequence[int]) -> None:
        """Overwrite pages (of every stop of a group, all they hold) with NaN: a
        debugging aid; a later read of a page's stale content then shows in the
        logits instead of passing for data."""
        if not pages:
            return
        index = torch.tensor(list(pages), dtype=torch.long, device=self.device)
        axis = 1 + self.manager.paged_groups[group].need.page_axis
        self.paged[group].index_fill_(axis, index, float("nan"))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.paged + self.state)


def kv_bytes_per_token(manager_needs, kv_dtype: torch.dtype) -> int:
    """Bytes one token costs over all stops that keep something per token
    (sizing the pool from free memory, cf. python/freetoken/kvcache/mha_pool.py:85-94)."""
    from .manager import PerTokenNeed
    total = 0
    for need in manager_needs:
        if isinstance(need, PerTokenNeed):
            dtype = kv_dtype if need.storage_dtype is None else _STATE_DTYPES[need.storage_dtype]
            total += need.elements_per_token() * torch.empty((), dtype=dtype).element_size()
    return total
