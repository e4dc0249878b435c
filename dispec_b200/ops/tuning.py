"""Launch-shape choices of the kernels, in one place, keyed by quantities of the launch (bytes,
rows, resident CTA slots, keys per CTA) and by the device's SM count, never by a model.

Every constant says what was measured.  None of them bears on correctness: the kernels take any
value that passes their own argument checks and give the same result bit for bit, except where
a split count changes the order of a 32-bit sum.
"""
from __future__ import annotations

import torch

_sm_count: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_count:
        _sm_count[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_count[index]


# ---- few-row matrix product (gemm_stream.cu) ------------------------------------------------
# Its CTAs keep about 100 KB of W on their way each, so two are resident per SM (the second slot is
# for the next kernel's CTAs, which fill their rings while this kernel drains).  K is split over a
# cluster until the launch has one CTA per SM; measured at 8 and at 64 rows: splitting further, to
# both resident slots, is slower (the gate/up product of 140 blocks cut in two: 8 % on the whole step).
STREAM_CTAS_PER_SM = 1


def stream_target_ctas(device=None) -> int:
    return STREAM_CTAS_PER_SM * sm_count(device)


# A product that streams at least this many bytes of W lets its successor start (programmatic
# dependent launch) only once its last tile of W is requested: what the successor requests before
# its own wait would otherwise compete with a long stream.  Shorter products let it start at once.
# Measured on captured decode steps, 8 rows: products of 4.7 to 6.3 MB are faster with the early
# trigger, products of 27 MB and more with the late one (1.334 -> 1.312 ms a step at 28 layers).
STREAM_LATE_TRIGGER_BYTES = 16 << 20

# A product of a few hundred rows: the many-row kernel cuts it into tiles of 256 rows x 192 or 256
# columns and does not split K, so a narrow product with a long K (down_proj: 8 tiles of 140 k
# blocks) keeps a tenth of the SMs busy; the few-row kernel run once per 128 rows streams W again for
# every chunk but fills the SMs.  Estimates in microseconds, fitted on captured decode steps of the
# 1.5B sizes (qkv / o_proj / gate_up / down: 13 / 14 / 18 / 45 us as one many-row product at 128 to
# 256 rows; 8.9 / 9.0 / 16.3 / 14.2 us per chunk of 128 rows): whichever is smaller runs.
MANY_ROW_US_PER_K_BLOCK = 0.31   # one tile's k block of 64 on a CTA pair that streams alone
MANY_ROW_US_FIXED = 6.0
CHUNK_US_FIXED = 8.0
CHUNK_BYTES_PER_US = 4.5e6       # W bytes a microsecond of the few-row kernel at 128 rows


def rows_in_chunks_is_faster(M: int, N: int, K: int, device=None, chunk_rows: int = 128) -> bool:
    """Whether ceil(M / chunk_rows) launches of the few-row product beat one many-row product."""
    pairs = max(1, sm_count(device) // 2)
    width = 256
    tiles = -(-M // 256) * -(-N // width)
    many = MANY_ROW_US_FIXED + -(-tiles // pairs) * -(-K // 64) * MANY_ROW_US_PER_K_BLOCK
    many = max(many, 2.0 * N * K / 6.5e6)
    chunks = -(-M // chunk_rows)
    return chunks * (CHUNK_US_FIXED + 2.0 * N * K / CHUNK_BYTES_PER_US) < many


# ---- attention of single tokens (attn_mma.cu, decode kernel) ---------------------------------
ATTN_CTAS_PER_SM = 2  # resident CTAs the decode launch aims for
CLUSTER_MAX_SPLITS = 8  # key splits of one row that merge on chip (one thread-block cluster)
SPLIT_MIN_KEYS = 256  # a split is not worth less than this many keys
MAX_OUTER = 32  # key ranges per row beyond the cluster
OUTER_MIN_KEYS = 256  # a CTA of a row cut into ranges still reads at least this many keys
MAX_SPLITS = 32  # splits merged from global scratch (groups too large for the cluster kernels)


def attention_target_ctas(device=None) -> int:
    return ATTN_CTAS_PER_SM * sm_count(device)


def choose_splits(num_rows: int, num_kv_heads: int, max_ctx: int, target_ctas: int,
                  limit: int = CLUSTER_MAX_SPLITS) -> int:
    """Key splits for single-token rows so that rows x KV heads x splits covers ``target_ctas``
    (``attention_target_ctas(device)``) once, each split keeping at least ``SPLIT_MIN_KEYS`` keys.  Measured at 1,100 keys and
    128-wide heads, 2 KV heads: the best count keeps the launch within two CTAs per SM (8 splits
    at 8 rows, 4 at 32, 2 at 64, 1 at 128)."""
    if num_rows <= 0:
        return 1
    want = max(1, target_ctas // (num_rows * num_kv_heads))
    return max(1, min(want, limit, -(-max_ctx // SPLIT_MIN_KEYS)))


def choose_outer(num_rows: int, num_kv_heads: int, max_ctx: int, splits: int, target_ctas: int) -> int:
    """Key ranges per single-token row on top of the cluster's ``splits``: when a full cluster
    per row and KV head still leaves SMs idle (few rows) and the context is long enough to share.
    Measured at 128-wide heads: the best count brings the launch to about two CTAs per SM (16
    ranges for one row of 32,768 keys, 2 for 8 rows), as long as a CTA keeps ``OUTER_MIN_KEYS``."""
    if num_rows <= 0 or splits < CLUSTER_MAX_SPLITS:
        return 1
    want = target_ctas // (num_rows * num_kv_heads * splits)
    return max(1, min(want, MAX_OUTER, max_ctx // (splits * OUTER_MIN_KEYS)))
