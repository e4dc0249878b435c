"""Argmax and temperature / top-k / top-p sampling kernels over 32-bit logits."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit per row; ties go to the lowest index.  int32 [n]."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2
    assert logits.stride(1) == 1
    n, v = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    # a large vocabulary is cut into chunks so that a few rows still fill the SMs
    chunks = 1 if v < 16384 else max(1, min(v // 4096, 64))
    if chunks > 1:
        part_val = torch.empty((n, chunks), dtype=torch.float32, device=logits.device)
        part_idx = torch.empty((n, chunks), dtype=torch.int32, device=logits.device)
    else:
        part_val = part_idx = None
    L.check(L.core().dsp_argmax(L.ptr(logits), L.i64(logits.stride(0)), n, v, L.ptr(out), chunks,
                                L.ptr(part_val), L.ptr(part_idx), L.stream_handle()),
            launches=2 if chunks > 1 else 1)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row.  temperature[r] <= 0: argmax; top_k[r] == 0 and top_p[r] >= 1: masks
    off; uniform[r] in [0, 1) drives the inverse-CDF draw in vocabulary order."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2
    assert logits.stride(1) == 1
    n, v = logits.shape
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (uniform, torch.float32)):
        assert t.is_cuda and t.dtype == dt and t.shape == (n,) and t.is_contiguous()
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    L.check(L.core().dsp_sample(L.ptr(logits), L.i64(logits.stride(0)), n, v, L.ptr(temperature),
                                L.ptr(top_k), L.ptr(top_p), L.ptr(uniform), L.ptr(out),
                                L.stream_handle()))
    return out
