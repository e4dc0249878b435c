"""Causal grouped-query attention over the paged key/value cache."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L

ROWS_PER_TILE = 64  # query rows (token, head-in-group pairs) one tensor-core tile holds


def tokens_per_tile(group_size: int) -> int | None:
    """Query tokens per tile of the tensor-core kernel (None: groups too large for it)."""
    if group_size > ROWS_PER_TILE:
        return None
    return ROWS_PER_TILE // group_size


def paged_attention_generic(q: torch.Tensor, q_stride: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            page_table: torch.Tensor, positions: torch.Tensor,
                            seq_of_token: torch.Tensor, out: torch.Tensor, num_heads: int,
                            num_kv_heads: int, head_dim: int, window: int, scale: float) -> torch.Tensor:
    """32-bit arithmetic kernel, any head size up to 512 and any group size.

    q: element (t, h, d) at q.data_ptr + (t * q_stride + h * D + d); out: [T, H * D].
    The query at absolute position p = positions[t] sees keys max(0, p-window+1)..p
    (window 0: from 0) of sequence seq_of_token[t].
    """
    assert q.is_cuda and k_pool.is_cuda, "CUDA tensors only (there is no CPU path)"
    T = positions.shape[0]
    num_pages, kvh, page_size, d = k_pool.shape
    assert (kvh, d) == (num_kv_heads, head_dim) and v_pool.shape == k_pool.shape
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.dtype == q.dtype
    assert out.is_contiguous() and out.shape == (T, num_heads * head_dim) and out.dtype == q.dtype
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    L.check(L.core().dsp_attn_generic(
        L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
        page_table.stride(0), L.ptr(positions), L.ptr(seq_of_token), L.ptr(out),
        L.i64(out.stride(0)), T, num_heads, num_kv_heads, head_dim, page_size, num_pages,
        window, L.f32(scale), L.dtype_code(q.dtype), L.stream_handle()))
    return out


def paged_attention(ctx, q: torch.Tensor, q_stride: int, cache, out: torch.Tensor, num_heads: int,
                    num_kv_heads: int, head_dim: int, window: int, scale: float) -> torch.Tensor:
    """Attention of the step described by ``ctx`` over the layer cache ``cache``."""
    return paged_attention_generic(q, q_stride, cache.key_pool, cache.value_pool, cache.page_table,
                                   ctx.positions, ctx.seq_of_token, out, num_heads, num_kv_heads,
                                   head_dim, window, scale)
