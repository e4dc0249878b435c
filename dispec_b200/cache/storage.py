"""Device memory behind the cache manager: one key/value pool per cache group and one
buffer per kind of fixed-size per-request state.

Pool layout: ``[layer cache, K|V, page, kv head, offset in page, head_dim]``, so that the
``page_size x head_dim`` tile of one head of one page is contiguous (one 4 KB box at
page 16, head 128, bfloat16).  The reference keeps ``[layer, slot, kv head, head_dim]``
(puneethgv/DiSpec dispec/kv/paged_cache.py:39-41).
"""
from __future__ import annotations

import torch

from dispec_b200.cache.manager import CacheGroupSpec


class CacheStorage:
    def __init__(self, groups: list[CacheGroupSpec], page_size: int, num_pages: list[int],
                 dtype: torch.dtype, device, poison: bool = False):
        self.page_size = page_size
        self.dtype = dtype
        self.pools: list[torch.Tensor] = []
        for spec, n in zip(groups, num_pages):
            shape = (spec.num_slots, 2, n, spec.num_kv_heads, page_size, spec.head_dim)
            pool = torch.empty(shape, dtype=dtype, device=device)
            # the reference zero-fills (dispec/kv/paged_cache.py:39-41); NaN on request, so that a
            # read of a never-written or stale slot shows in tests
            pool.fill_(float("nan") if poison else 0.0)
            self.pools.append(pool)

    def key_pool(self, group: int, slot: int) -> torch.Tensor:
        return self.pools[group][slot, 0]

    def value_pool(self, group: int, slot: int) -> torch.Tensor:
        return self.pools[group][slot, 1]

    def poison_pages(self, group: int, pages: list[int]) -> None:
        if pages:
            idx = torch.tensor(pages, device=self.pools[group].device, dtype=torch.long)
            self.pools[group][:, :, idx] = float("nan")

    def memory_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools)


class StateStorage:
    """``[max_num_seqs, *shape]`` per state need, indexed by a request's state slot."""

    def __init__(self, needs: list, max_num_seqs: int, device):
        self.buffers: list[torch.Tensor] = []
        for need in needs:
            dt = {"float32": torch.float32, "int32": torch.int32, "bfloat16": torch.bfloat16}[need.dtype]
            self.buffers.append(torch.zeros((max_num_seqs,) + tuple(need.shape), dtype=dt, device=device))

    def reset_slot(self, slot: int) -> None:
        for b in self.buffers:
            b[slot].zero_()
