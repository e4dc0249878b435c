"""Causal grouped-query attention over the paged key/value cache."""
from __future__ import annotations

import ctypes

import torch

from dispec_b200.ops import library as L
from dispec_b200.ops import tuning
from dispec_b200.ops.tuning import CLUSTER_MAX_SPLITS

ROWS_PER_TILE = 64  # query rows (token, head-in-group pairs) one tensor-core tile holds
PREFILL_ROWS_PER_TILE = 128  # rows of a tile of the tcgen05 kernel for portions of prompts
DECODE_KERNEL_MAX_GROUP = 16  # query heads per KV head the warp-parallel single-token kernel holds


def tokens_per_tile(group_size: int) -> int | None:
    """Query tokens per tile of the tensor-core kernel (None: groups too large for it)."""
    if group_size > ROWS_PER_TILE:
        return None
    return ROWS_PER_TILE // group_size


def prefill_tokens_per_tile(group_size: int) -> int:
    """Query tokens per tile of the tcgen05 kernel for portions of prompts."""
    return PREFILL_ROWS_PER_TILE // group_size


def tcgen05_supported(head_dim: int, group_size: int, page_size: int, dtype: torch.dtype) -> bool:
    """The tcgen05 kernel is built for head sizes 64 and 128 and pages of 8 to 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128)
            and group_size <= ROWS_PER_TILE and page_size in (8, 16, 32, 64))


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


_MMA_ERRORS = {1: "launch failed", 2: "unsupported head/group/split counts",
               3: "operands must be 16-byte aligned with strides in whole 16-byte pieces",
               4: "shared memory opt-in failed"}
_partials: dict = {}
_retired: list = []
_err_addr: dict = {}


def tensor_core_supported(head_dim: int, group_size: int, dtype: torch.dtype) -> bool:
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and group_size <= ROWS_PER_TILE)


def _partial_buffers(device, rows: int, splits: int, head_dim: int):
    """Scratch for split attention: unnormalised outputs and (max, sum) per row and split."""
    key = torch.device(device).index or 0
    need = rows * splits * (head_dim + 2)
    buf = _partials.get(key)
    if buf is None or buf.numel() < need:
        # a captured step keeps the address of the scratch it was captured with: a buffer that is
        # outgrown stays alive (sizes at least double, so all of them together stay below twice the last)
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(max(need, 1 << 20, 2 * (buf.numel() if buf is not None else 0)),
                          dtype=torch.float32, device=device)
        _partials[key] = buf
    n_o = rows * splits * head_dim
    return buf[:n_o], buf[n_o:n_o + rows * splits * 2]


def reserve_partials(device, rows: int, splits: int, head_dim: int) -> None:
    """Sizes the scratch ahead of time (before a CUDA graph is captured)."""
    _partial_buffers(device, rows, splits, head_dim)


def _device_error_address(device) -> int:
    key = torch.device(device).index or 0
    if key not in _err_addr:
        fn = L.core().dsp_device_error_address
        fn.restype = ctypes.c_ulonglong
        _err_addr[key] = int(fn())
    return _err_addr[key]


def choose_splits(num_decode_tiles: int, num_kv_heads: int, max_ctx: int, device=None) -> int:
    """Key splits for single-token rows on this device (see ``tuning.choose_splits``)."""
    return tuning.choose_splits(num_decode_tiles, num_kv_heads, max_ctx, tuning.attention_target_ctas(device))


def choose_outer(num_decode_tiles: int, num_kv_heads: int, max_ctx: int, splits: int, device=None) -> int:
    """Key ranges per single-token row beyond the cluster (see ``tuning.choose_outer``)."""
    return tuning.choose_outer(num_decode_tiles, num_kv_heads, max_ctx, splits,
                               tuning.attention_target_ctas(device))


def decode_rope_fusable(ctx, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                        dtype: torch.dtype) -> bool:
    """Whether the single tokens of this step go through the kernel that rotates q and k itself
    (then the separate rotation kernel must skip them)."""
    group = num_heads // num_kv_heads
    return (ctx.num_decode_seqs > 0 and tensor_core_supported(head_dim, group, dtype)
            and group <= DECODE_KERNEL_MAX_GROUP and tokens_per_tile(group) in ctx.attention_tiles
            and 0 < rotary_dim <= head_dim and rotary_dim % 16 == 0)


def _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                tile_offset, num_tiles, out, part_o, part_ml, H, KVH, D, tpt, window, splits, scale,
                cluster_combine=False, decode_only=False, fused_rope=None, outer=1):
    num_pages, _, page_size, _ = k_pool.shape
    lib = L.attention_library(D)
    fn = getattr(lib, f"dsp_attn_mma_d{D}")
    rc = fn(L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
            page_table.stride(0), L.ptr(q_start), L.ptr(ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0),
            tile_offset, num_tiles, L.ptr(out), L.i64(out.stride(0)), L.ptr(part_o), L.ptr(part_ml),
            H, KVH, tpt, page_size, num_pages, window, splits, int(cluster_combine), int(decode_only),
            outer, L.f32(scale), L.ptr(fused_rope[0]) if fused_rope else None, fused_rope[1] if fused_rope else 0,
            1 if fused_rope else 0, int(fused_rope[2]) if fused_rope else 0,
            ctypes.c_void_p(_device_error_address(q.device)), L.stream_handle())
    L.LaunchCounter.n += 1
    if rc != 0:
        raise L.KernelError(f"dsp_attn_mma_d{D}: {_MMA_ERRORS.get(rc, rc)}")


def _launch_tcgen05(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                    tile_offset, num_tiles, out, H, KVH, D, tpt, window, scale):
    num_pages, _, page_size, _ = k_pool.shape
    lib = L.prefill_attention_library(D)
    fn = getattr(lib, f"dsp_attn_tcgen05_d{D}")
    rc = fn(L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
            page_table.stride(0), L.ptr(q_start), L.ptr(ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0),
            tile_offset, num_tiles, L.ptr(out), L.i64(out.stride(0)), H, KVH, tpt, page_size, num_pages,
            window, L.f32(scale), ctypes.c_void_p(_device_error_address(q.device)), L.stream_handle())
    L.LaunchCounter.n += 1
    if rc != 0:
        raise L.KernelError(f"dsp_attn_tcgen05_d{D}: {_TCGEN05_ERRORS.get(rc, rc)}")


_TCGEN05_ERRORS = {1: "launch failed", 2: "unsupported head/group counts or page size",
                   3: "operands must be 16-byte aligned with strides in whole 16-byte pieces",
                   4: "shared memory opt-in or tensor map creation failed"}


def paged_attention_tiles(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                          tile_tok0, num_tiles, num_decode_tiles, out, H, KVH, D, window, scale,
                          splits: int, prefill_tiles=None, fused_rope=None, outer: int = 1,
                          decode_kernel: bool | None = None) -> torch.Tensor:
    """Tensor-core attention over a tile list whose first ``num_decode_tiles`` tiles are single
    tokens (run with ``splits`` key splits and merged), the rest portions of prompts.  With
    ``prefill_tiles`` = (tile_seq, tile_tok0, num_tiles) of the 128-row tiling (single tokens
    first as well) the portions of prompts run on the tcgen05 kernel.  ``fused_rope`` = (inv_freq,
    rotary_dim, write_kv): ``q`` are the fused q/k/v rows and the single tokens' rows are not
    rotated yet; their kernel rotates them and stores key and value (see ``decode_rope_fusable``).
    ``outer`` > 1 cuts each single token's keys into that many ranges, each run by a cluster of
    ``splits`` CTAs; a second kernel merges the ranges (long contexts at small batches).
    ``decode_kernel``: whether single tokens take the warp-parallel kernel (default: whenever
    the group of query heads per KV head fits it) or the tile kernel."""
    assert q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous()
    tpt = tokens_per_tile(H // KVH)
    group = H // KVH
    if decode_kernel is None:
        decode_kernel = group <= DECODE_KERNEL_MAX_GROUP
    decode_kernel = decode_kernel and group <= DECODE_KERNEL_MAX_GROUP
    if num_decode_tiles > 0:
        if splits <= CLUSTER_MAX_SPLITS and (decode_kernel or splits > 1):
            # single tokens: the cluster kernels (warp-parallel keys when the group fits 16 rows)
            if outer > 1 and not decode_kernel:
                outer = 1
            part_o = part_ml = None
            if outer > 1:
                part_o, part_ml = _partial_buffers(q.device, num_decode_tiles * H, outer, D)
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, part_o, part_ml, H, KVH, D, tpt, window,
                        splits, scale, cluster_combine=splits > 1, decode_only=decode_kernel,
                        fused_rope=fused_rope, outer=outer)
            if outer > 1:
                L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out),
                                                  L.i64(out.stride(0)), num_decode_tiles, H, D, outer,
                                                  L.dtype_code(out.dtype), L.stream_handle()))
        elif fused_rope:
            raise L.KernelError("single tokens were left unrotated for a kernel that is not in use")
        elif splits > 1:
            rows = num_decode_tiles * H  # decode tokens are the first rows of the flat batch
            part_o, part_ml = _partial_buffers(q.device, rows, splits, D)
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, part_o, part_ml, H, KVH, D, tpt, window,
                        splits, scale)
            L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out),
                                              L.i64(out.stride(0)), num_decode_tiles, H, D, splits,
                                              L.dtype_code(out.dtype), L.stream_handle()))
        else:
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, None, None, H, KVH, D, tpt, window, 1, scale)
    if prefill_tiles is not None:
        big_seq, big_tok0, big_n = prefill_tiles
        if big_n > num_decode_tiles:
            _launch_tcgen05(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, big_seq, big_tok0,
                            num_decode_tiles, big_n - num_decode_tiles, out, H, KVH, D,
                            prefill_tokens_per_tile(H // KVH), window, scale)
    elif num_tiles > num_decode_tiles:
        _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                    num_decode_tiles, num_tiles - num_decode_tiles, out, None, None, H, KVH, D, tpt,
                    window, 1, scale)
    return out


def paged_attention_tensor_core(q, q_stride, k_pool, v_pool, page_table, positions, seq_of_token, out,
                                num_heads, num_kv_heads, head_dim, window, scale, q_lens, ctx_lens,
                                splits=None, decode_kernel=None, prefill_kernel=None) -> torch.Tensor:
    """Stand-alone form (tests, tools): builds the tile list for sequences given by their
    ``q_lens`` and ``ctx_lens`` (single-token sequences must come first).  ``prefill_kernel``
    "mma" keeps portions of prompts on the mma.sync kernel where the tcgen05 kernel would take
    them; ``decode_kernel`` False keeps single tokens on the tile kernel."""
    dev_ = q.device
    group = num_heads // num_kv_heads
    tpt = tokens_per_tile(group)

    def tile_list(per_tile):
        ts, t0, n_dec = [], [], 0
        for s, n in enumerate(q_lens):
            if n == 1 and n_dec == s:
                n_dec += 1
            for a in range(0, n, per_tile):
                ts.append(s)
                t0.append(a)
        return ts, t0, n_dec

    ts, t0, n_dec = tile_list(tpt)
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev_)
    if splits is None:
        splits = choose_splits(n_dec, num_kv_heads, max(ctx_lens), q.device)
    prefill_tiles = None
    if prefill_kernel != "mma" and tcgen05_supported(head_dim, group, k_pool.shape[2], q.dtype):
        bs, b0, _ = tile_list(prefill_tokens_per_tile(group))
        prefill_tiles = (i32(bs), i32(b0), len(bs))
    return paged_attention_tiles(q, q_stride, k_pool, v_pool, page_table, i32(starts), i32(ctx_lens),
                                 i32(ts), i32(t0), len(ts), n_dec, out, num_heads, num_kv_heads,
                                 head_dim, window, scale, splits, prefill_tiles, decode_kernel=decode_kernel)


def paged_attention(ctx, q: torch.Tensor, q_stride: int, cache, out: torch.Tensor, num_heads: int,
                    num_kv_heads: int, head_dim: int, window: int, scale: float, fused_rope=None) -> torch.Tensor:
    """Attention of the step described by ``ctx`` over the layer cache ``cache``: the
    tensor-core kernel for bfloat16 where it is built for the sizes, the 32-bit kernel
    otherwise (and always on the float32 path)."""
    group = num_heads // num_kv_heads
    tpt = tokens_per_tile(group)
    if tensor_core_supported(head_dim, group, q.dtype) and tpt in ctx.attention_tiles:
        tile_seq, tile_tok0, num_tiles = ctx.attention_tiles[tpt]
        splits = ctx.decode_splits if ctx.decode_splits else choose_splits(
            ctx.num_decode_seqs, num_kv_heads, ctx.max_ctx_len, q.device)
        outer = ctx.decode_outer if ctx.decode_outer else choose_outer(
            ctx.num_decode_seqs, num_kv_heads, ctx.max_ctx_len, splits, q.device)
        prefill_tiles = None
        big = prefill_tokens_per_tile(group)
        if big in ctx.attention_tiles and tcgen05_supported(head_dim, group, cache.key_pool.shape[2], q.dtype):
            prefill_tiles = ctx.attention_tiles[big]
        return paged_attention_tiles(q, q_stride, cache.key_pool, cache.value_pool, cache.page_table,
                                     ctx.q_start, ctx.ctx_len, tile_seq, tile_tok0, num_tiles,
                                     ctx.num_decode_seqs, out, num_heads, num_kv_heads, head_dim,
                                     window, scale, splits, prefill_tiles, fused_rope, outer)
    if fused_rope:
        raise L.KernelError("single tokens were left unrotated for a kernel that is not in use")
    return paged_attention_generic(q, q_stride, cache.key_pool, cache.value_pool, cache.page_table,
                                   ctx.positions, ctx.seq_of_token, out, num_heads, num_kv_heads,
                                   head_dim, window, scale)
