"""Embedding gather, RMSNorm (plain and fused with the residual sum), SwiGLU, and the rotary
rotation fused with the paged key/value write."""
from __future__ import annotations

import ctypes

import torch

from dispec_b200.ops import library as L


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise L.KernelError("kernel inputs must be CUDA tensors (there is no CPU path)")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32."""
    _cuda(table, ids)
    assert ids.dtype == torch.int32 and ids.is_contiguous() and table.is_contiguous()
    n, hidden = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty((n, hidden), dtype=table.dtype, device=table.device)
    L.check(L.core().dsp_embed(L.ptr(table), L.ptr(ids), L.ptr(out), n, hidden, table.shape[0],
                               L.dtype_code(table.dtype), L.stream_handle()))
    return out


def feed_tokens(ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """ids[t] = prev[src[t]] where src[t] >= 0 (all int32, on the device): tokens sampled in the
    previous step become inputs of this one without passing through the host."""
    _cuda(ids, src, prev)
    assert ids.dtype == src.dtype == prev.dtype == torch.int32
    assert ids.is_contiguous() and src.is_contiguous() and prev.is_contiguous()
    assert src.shape[0] <= ids.shape[0]
    L.check(L.core().dsp_feed_tokens(L.ptr(ids), L.ptr(src), L.ptr(prev), src.shape[0], prev.shape[0],
                                     L.stream_handle()))


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: torch.Tensor | None = None,
             rows: torch.Tensor | None = None, write_back: bool = False,
             out: torch.Tensor | None = None) -> torch.Tensor:
    """y = w * round(x * rsqrt(mean(x^2) + eps)), 32-bit inside.

    ``delta``: the norm is of round(x + delta); ``write_back`` stores that sum into x.
    ``rows`` (int32) gathers input rows; the output is dense.
    """
    _cuda(x, weight, delta, rows)
    assert x.dim() == 2 and x.is_contiguous() and weight.dtype == x.dtype
    hidden = x.shape[1]
    assert weight.shape == (hidden,)
    if delta is not None:
        assert delta.shape == x.shape and delta.dtype == x.dtype and delta.is_contiguous()
    n = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        assert rows.dtype == torch.int32 and not write_back
    if out is None:
        out = torch.empty((n, hidden), dtype=x.dtype, device=x.device)
    L.check(L.core().dsp_rmsnorm(L.ptr(x), L.ptr(delta), L.ptr(weight), L.ptr(out), L.ptr(rows), n,
                                 hidden, ctypes.c_float(eps), int(write_back),
                                 L.dtype_code(x.dtype), L.stream_handle()))
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int = 0) -> torch.Tensor:
    """out[t, i] = silu(gate(t, i)) * up(t, i).  ``block`` 0: a row is [gates | ups]; b > 0: gates
    and ups alternate in blocks of b columns (b gates, their b ups, the next b gates, ...)."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    n, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    L.check(L.core().dsp_swiglu(L.ptr(gate_up), L.ptr(out), n, inter, block, L.dtype_code(gate_up.dtype),
                                L.stream_handle()))
    return out


def rope_kv_store(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  page_table: torch.Tensor, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
                  inv_freq: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int, write_kv: bool = True) -> None:
    """Rotates q and k inside ``qkv`` [T, (H + 2 KVH) D] in place and writes k, v to the pools
    [num_pages, KVH, page_size, D] at page_table[seq, pos // page_size], offset pos % page_size.
    Rows with a negative position are skipped."""
    _cuda(qkv, positions, seq_of_token, page_table, k_pool, v_pool, inv_freq)
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    if write_kv:
        assert k_pool is not None and v_pool is not None
        assert k_pool.dtype == qkv.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
        num_pages, kvh, page_size, d = k_pool.shape
        assert (kvh, d) == (num_kv_heads, head_dim) and v_pool.shape == k_pool.shape
    else:
        num_pages, page_size = 0, 1
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype == torch.float32
        assert inv_freq.shape[0] >= rotary_dim // 2
    L.check(L.core().dsp_rope_kv_store(
        L.ptr(qkv), L.ptr(positions), L.ptr(seq_of_token), L.ptr(page_table), page_table.stride(0),
        L.ptr(k_pool), L.ptr(v_pool), L.ptr(inv_freq), T, num_heads, num_kv_heads, head_dim,
        rotary_dim, page_size, num_pages, int(write_kv), L.dtype_code(qkv.dtype), L.stream_handle()))


def fill_normal(out: torch.Tensor, seed: int, ordinal: int, std: float, mean: float = 0.0,
                through_bf16: bool = False) -> torch.Tensor:
    """out.flatten()[i] = mean + std * z(seed, ordinal, i): the counter-based normal numbers of
    ``dispec_b200.weights.counter_rng`` (same bits), rounded once to out's type (float32 or
    bfloat16).  ``through_bf16`` rounds to bfloat16 first even when out is float32."""
    _cuda(out)
    assert out.is_contiguous() and 0 <= ordinal < (1 << 32) and 0 <= seed < (1 << 64)
    with torch.cuda.device(out.device):
        L.check(L.core().dsp_fill_normal(L.ptr(out), L.i64(out.numel()), ctypes.c_ulonglong(seed),
                                         ctypes.c_uint(ordinal), ctypes.c_float(mean), ctypes.c_float(std),
                                         L.dtype_code(out.dtype), int(through_bf16), L.stream_handle()))
    return out
