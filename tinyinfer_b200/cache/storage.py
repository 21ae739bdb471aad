"""Device memory behind the page ids: for every cache entry that wants pages one tensor
[2, pages, kv_heads, page_size, head_dim] (keys then values; one (page, head) tile of
page_size x head_dim is contiguous, which is what a tiled copy wants), and for every entry that
wants per-request state one tensor [slots, *shape].

The reference allocates [layers, 2, blocks, block_size, heads, dim] in one piece
(tinyinfer/layers/attention.py:103-120); splitting by entry lets groups differ in every size.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .manager import CacheManager


def bytes_per_page(needs, page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs across all cache entries of all groups (they share the count)."""
    total = 0
    for need, _state in needs:
        if need is not None:
            total += 2 * need.num_kv_heads * page_size * need.head_dim * dtype.itemsize
    return total


class CacheStorage:
    def __init__(self, needs, manager: CacheManager, dtype: torch.dtype, device, poison: bool = False):
        self.dtype = dtype
        self.device = torch.device(device)
        self.kv: List[Optional[torch.Tensor]] = []
        self.state: List[Optional[torch.Tensor]] = []
        for entry, (need, state) in enumerate(needs):
            if need is None:
                self.kv.append(None)
            else:
                # one page more than the pool hands out: the last one takes the keys of the padding rows
                # that fill a decode batch up to the size of its captured graph (see dump_page)
                pages = manager.groups[manager.group_of_entry[entry]].pool.num_pages + 1
                shape = (2, pages, need.num_kv_heads, manager.page_size, need.head_dim)
                t = torch.empty(shape, dtype=dtype, device=self.device)
                # tests poison the pool: a read outside a request's own keys then shows as NaN
                t.fill_(float("nan") if poison else 0.0)
                self.kv.append(t)
            if state is None:
                self.state.append(None)
            else:
                # one slot more than requests can hold: the padding rows' (see dump_slot)
                self.state.append(torch.zeros((manager.max_requests + 1, *state.shape),
                                              dtype=state.dtype, device=self.device))

    @staticmethod
    def dump_page(manager: CacheManager, group: int) -> int:
        """The page id no request ever holds: padding rows write their keys and values there."""
        return manager.groups[group].pool.num_pages

    @staticmethod
    def dump_slot(manager: CacheManager) -> int:
        """The state slot no request ever holds: a mixer that updates its state on the device, for
        every row of the step alike, updates this one for the padding rows."""
        return manager.max_requests

    def reset_state_slot(self, slot: int) -> None:
        for t in self.state:
            if t is not None:
                t[slot].zero_()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + self.state if t is not None)
