"""Device memory behind the cache manager: per cache group one pool for each tensor the
group's mixers keep per token (a key and a value for ordinary attention; any other named
tensors, each with its own heads and width, for another mixer), and one buffer per kind of
fixed-size per-request state.

Pool layout: ``[layer cache, page, head, offset in page, width]``, so that the
``page_size x width`` tile of one head of one page is contiguous (one 4 KB box at page 16,
head size 128, bfloat16).  The reference keeps ``[layer, slot, kv head, head_dim]``
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
        self.pools: list[dict[str, torch.Tensor]] = []  # per group: tensor name -> pool
        for spec, n in zip(groups, num_pages):
            named = {}
            for t in spec.tensors:
                pool = torch.empty((spec.num_slots, n, t.num_heads, page_size, t.width), dtype=dtype, device=device)
                # the reference zero-fills (dispec/kv/paged_cache.py:39-41); NaN on request, so that a
                # read of a never-written or stale slot shows in tests
                pool.fill_(float("nan") if poison else 0.0)
                named[t.name] = pool
            self.pools.append(named)

    def layer_tensors(self, group: int, slot: int) -> dict:
        """name -> ``[page, head, offset in page, width]`` of one layer cache."""
        return {name: pool[slot] for name, pool in self.pools[group].items()}

    def poison_pages(self, group: int, pages: list[int]) -> None:
        if pages:
            for pool in self.pools[group].values():
                idx = torch.tensor(pages, device=pool.device, dtype=torch.long)
                pool[:, idx] = float("nan")

    def memory_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for named in self.pools for p in named.values())


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
