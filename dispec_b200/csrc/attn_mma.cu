// Causal grouped-query attention over the paged cache on the tensor cores, bfloat16 in, 32-bit
// softmax and accumulation.  Compiled once per head size (-DDSP_HEAD_DIM=...).
//
// A tile is 64 query rows of one KV head of one sequence; a row is a (token, head-in-group)
// pair, so the G query heads that share a KV head share every key/value load, and a single
// decoded token fills G rows.  Keys are walked in tiles of 64 through the page table
// (cp.async, two stages).  S = Q K^T and O += P V are mma.m16n8k16; the softmax is the online
// form (running max and sum per row, base 2).  The query at position p sees keys b with
// max(0, p - window + 1) <= b <= p.  With num_splits > 1 the key tiles of a query tile are
// divided among grid.z CTAs, each producing an unnormalised partial (o, m, l) per row.  With up to
// 8 splits those CTAs form a thread-block cluster and merge their partials through distributed
// shared memory (each CTA finishes a share of the rows, reading every rank's partial in rank
// order); with more splits the partials go to global scratch and a second kernel
// (dsp_attn_combine) merges them.
//
// Shared memory rows are 16-byte pieces XOR-swizzled by the row index, so ldmatrix reads are
// conflict-free for head sizes of 64 and above.  Keys at or beyond the sequence length, and keys
// on pages that were given back, are zero-filled, never read.
#include <cooperative_groups.h>

#include "tcgen05_common.cuh"  // bounded mbarrier waits, cluster addresses, counted remote stores

namespace cg = cooperative_groups;

#ifndef DSP_HEAD_DIM
#error "compile with -DDSP_HEAD_DIM=<head size>"
#endif

#define DSP_CAT2(a, b) a##b
#define DSP_CAT(a, b) DSP_CAT2(a, b)

namespace {
constexpr int D = DSP_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int BM = 64, BN = 64, THREADS = 128;
constexpr int CHUNKS = D / 8;  // 16-byte pieces per row
constexpr int ROW_CHUNKS = CHUNKS <= 2 ? 2 : CHUNKS <= 4 ? 4 : ((CHUNKS + 7) / 8) * 8;
constexpr int SW_MASK = (ROW_CHUNKS < 8 ? ROW_CHUNKS : 8) - 1;
constexpr int ROW_BYTES = ROW_CHUNKS * 16;
constexpr int TILE_BYTES = 64 * ROW_BYTES;

// Timestamps of the single-token kernel for measurements, compiled in only with -DDSP_STAMPS.
#ifdef DSP_STAMPS
__device__ unsigned long long g_attn_stamps[1 << 20];
#define ASTAMP(pt)                                                                                            \
  do {                                                                                                        \
    if (p.stamp_base >= 0) {                                                                                  \
      unsigned long long t__;                                                                                 \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                                 \
      g_attn_stamps[(size_t)p.stamp_base +                                                                    \
                    (((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 12 + (pt)] = t__; \
    }                                                                                                         \
  } while (0)
#else
#define ASTAMP(pt)
#endif

struct Params {
  long stamp_base;
  const bf16* q;
  long q_stride;
  const bf16* k_pool;
  const bf16* v_pool;
  const int* page_table;
  int pt_stride;
  const int* q_start;
  const int* ctx_len;
  const int* tile_seq;
  const int* tile_tok0;
  bf16* out;
  long out_stride;
  float* part_o;   // [(t * H + h) * splits + split][D]
  float* part_ml;  // [(t * H + h) * splits + split][2]
  int H, KVH, G, tokens_per_tile, page_size, page_shift, num_pages, window, num_splits;
  int cluster_combine;  // the splits of a tile are one cluster and merge on chip
  float scale_log2;
  int* err;
  // single-token kernel only: q points into the fused q/k/v rows before rotation; the kernel rotates q
  // itself and, if write_kv, rotates the token's key, stores key and value into the cache and uses them
  const float* inv_freq;
  int rotary_dim, fused_rope, write_kv;
  // single-token kernel only: key ranges per row beyond the cluster (their partials go to part_o / part_ml)
  int num_outer, num_dec_tiles;
};

__device__ __forceinline__ uint32_t sw(int row, int chunk) {
  return (uint32_t)(row * ROW_BYTES + ((chunk ^ (row & SW_MASK)) << 4));
}
__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}
// the same for data that is read once per step (the cache's keys and values in decoding): its
// lines are the first to leave the L2
__device__ __forceinline__ void cp_async16_once(uint32_t smem, const void* gmem, bool valid, uint64_t policy) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(smem), "l"(gmem), "r"(bytes),
               "l"(policy));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS) attn_mma_kernel(const Params p, int tile_offset) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t s_base = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t q_s = s_base;
  const uint32_t k_s[2] = {s_base + TILE_BYTES, s_base + 2 * TILE_BYTES};
  const uint32_t v_s[2] = {s_base + 3 * TILE_BYTES, s_base + 4 * TILE_BYTES};

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g4 = lane >> 2, c4 = lane & 3;
  // later tiles of a prompt see more keys: the longest work is scheduled first
  const int tile = ((int)gridDim.x - 1 - (int)blockIdx.x) + tile_offset, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = p.tile_seq[tile], tok0 = p.tile_tok0[tile];
  const int qs = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - qs;
  const int ctx = p.ctx_len[seq];
  if (ctx <= 0 || q_len <= 0 || tok0 >= q_len) return;
  const int G = p.G;
  const int ntok = min(p.tokens_per_tile, q_len - tok0);
  const int nrows = ntok * G;
  const int pos0 = ctx - q_len + tok0;
  const int pos_last = pos0 + ntok - 1;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kt_begin = lo / BN, kt_end = pos_last / BN + 1;
  const int per = (kt_end - kt_begin + p.num_splits - 1) / p.num_splits;
  const int my_begin = kt_begin + split * per;
  const int my_end = min(kt_end, my_begin + per);
  const int* table = p.page_table + (size_t)seq * p.pt_stride;
  // set when a key tile met a page id outside the pool: from then on the mask looks every key's page
  // up again and hides the keys of such pages (their rows were zero-filled, not loaded)
  __shared__ int bad_page_seen;
  if (tid == 0) bad_page_seen = 0;
  __syncthreads();

  // ---- Q tile: two threads per row
  {
    const int r = tid >> 1, half = tid & 1;
    const bool valid = r < nrows;
    const bf16* src = p.q;
    if (valid) src = p.q + (size_t)(qs + tok0 + r / G) * p.q_stride + (size_t)(kvh * G + r % G) * D;
#pragma unroll
    for (int chunk = half; chunk < CHUNKS; chunk += 2) cp_async16(q_s + sw(r, chunk), src + chunk * 8, valid);
    cp_async_commit();
  }

  // two threads per key row: one page lookup per thread and tile, then 16-byte pieces of the row
  auto load_kv = [&](int kt, int buf) {
    const int r = tid >> 1, half = tid & 1;
    const int b = kt * BN + r;
    bool valid = b < ctx && b <= pos_last;
    size_t off = 0;
    if (valid) {
      const int lp = p.page_shift >= 0 ? (b >> p.page_shift) : (b / p.page_size);
      const int within = p.page_shift >= 0 ? (b & (p.page_size - 1)) : (b % p.page_size);
      const int page = table[lp];
      if (page < 0 || page >= p.num_pages) {
        if (b >= lo && half == 0) {
          atomicOr(p.err, DSP_ERR_BAD_PAGE);
          bad_page_seen = 1;
        }
        valid = false;
      } else {
        off = (((size_t)page * p.KVH + kvh) * p.page_size + within) * D;
      }
    }
#pragma unroll
    for (int chunk = half; chunk < CHUNKS; chunk += 2) {
      cp_async16(k_s[buf] + sw(r, chunk), p.k_pool + off + chunk * 8, valid);
      cp_async16(v_s[buf] + sw(r, chunk), p.v_pool + off + chunk * 8, valid);
    }
    cp_async_commit();
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int row0 = warp * 16 + g4, row1 = row0 + 8;
  const bool warp_active = warp * 16 < nrows;
  const int pos_r[2] = {pos0 + row0 / G, pos0 + row1 / G};
  const bool row_ok[2] = {row0 < nrows, row1 < nrows};

  if (my_begin < my_end) load_kv(my_begin, 0);
  for (int kt = my_begin; kt < my_end; ++kt) {
    const int buf = (kt - my_begin) & 1;
    if (kt + 1 < my_end) {
      load_kv(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_active) {
      float s[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
      const int m8 = lane >> 3, l8 = lane & 7;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, q_s + sw(warp * 16 + (m8 & 1) * 8 + l8, kk * 2 + (m8 >> 1)));
#pragma unroll
        for (int nn = 0; nn < BN / 16; ++nn) {
          uint32_t b[4];
          ldmatrix_x4(b, k_s[buf] + sw(nn * 16 + (m8 >> 1) * 8 + l8, kk * 2 + (m8 & 1)));
          mma_bf16(s[2 * nn], a, b[0], b[1]);
          mma_bf16(s[2 * nn + 1], a, b[2], b[3]);
        }
      }
      // mask, scale, online softmax
      const bool check_pages = bad_page_seen != 0;  // the same for the whole CTA (read after the barrier)
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int key = kt * BN + nt * 8 + 2 * c4 + (e & 1);
          bool vis = row_ok[r] && key <= pos_r[r] && (p.window == 0 || key > pos_r[r] - p.window);
          if (check_pages && vis) {
            const int page = table[key / p.page_size];
            vis = page >= 0 && page < p.num_pages;
          }
          const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
          s[nt][e] = v;
          tmax[r] = fmaxf(tmax[r], v);
        }
      float alpha[2], m_safe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
        const float m_new = fmaxf(m_run[r], tmax[r]);
        m_safe[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_safe[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[nt][e] - m_safe[e >> 1]);
          s[nt][e] = pv;
          l_run[e >> 1] += pv;
        }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int j = 0; j < BN / 16; ++j) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
        a[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
        a[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
        a[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
        for (int dd = 0; dd < D / 16; ++dd) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, v_s[buf] + sw(j * 16 + (m8 & 1) * 8 + l8, dd * 2 + (m8 >> 1)));
          mma_bf16(o[2 * dd], a, b[0], b[1]);
          mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  if (my_begin >= my_end) cp_async_wait<0>();

  // ---- epilogue
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (p.cluster_combine) {
    // partials of this CTA into its shared memory (the key/value tiles are no longer needed)
    __syncthreads();
    float* part_o = reinterpret_cast<float*>(smem);            // [64][D]
    float* part_ml = part_o + BM * D;                          // [64][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r == 0 ? row0 : row1;
      if (row < nrows) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<float2*>(part_o + row * D + i * 8 + 2 * c4) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
        if (c4 == 0) {
          part_ml[row * 2] = m_run[r];
          part_ml[row * 2 + 1] = l_run[r];
        }
      }
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int rank = (int)cluster.block_rank(), nsplit = p.num_splits;
    // rows are dealt to the CTAs of the cluster; a warp finishes one row at a time
    for (int row = rank * 4 + warp; row < nrows; row += nsplit * 4) {
      float M = -INFINITY;
      for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, cluster.map_shared_rank(part_ml, sp)[row * 2]);
      float L = 0.f;
      float acc[(D + 31) / 32];
#pragma unroll
      for (int j = 0; j < (D + 31) / 32; ++j) acc[j] = 0.f;
      for (int sp = 0; sp < nsplit; ++sp) {
        const float* ml = cluster.map_shared_rank(part_ml, sp);
        const float m = ml[row * 2];
        if (m == -INFINITY) continue;
        const float w = exp2f(m - M);
        L += w * ml[row * 2 + 1];
        const float* po = cluster.map_shared_rank(part_o, sp) + row * D;
#pragma unroll
        for (int j = 0; j < (D + 31) / 32; ++j) {
          const int d = lane + 32 * j;
          if (d < D) acc[j] += w * po[d];
        }
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      const size_t t = (size_t)qs + tok0 + row / G;
      bf16* dst = p.out + t * p.out_stride + (size_t)(kvh * G + row % G) * D;
#pragma unroll
      for (int j = 0; j < (D + 31) / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < D) dst[d] = __float2bfloat16(acc[j] * inv);
      }
    }
    cluster.sync();  // nobody leaves while its partials may still be read
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r == 0 ? row0 : row1;
    if (row >= nrows) continue;
    const size_t t = (size_t)qs + tok0 + row / G;
    const int h = kvh * G + row % G;
    if (p.num_splits == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      bf16* dst = p.out + t * p.out_stride + (size_t)h * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * c4) = v;
      }
    } else {
      const size_t idx = (t * p.H + h) * p.num_splits + split;
      float* dst = p.part_o + idx * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * c4) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
      if (c4 == 0) {
        p.part_ml[idx * 2] = m_run[r];
        p.part_ml[idx * 2 + 1] = l_run[r];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Single decoded tokens (the G rows of one KV head fit one 16-row mma tile), built for latency:
// a step's attention reads a few hundred KB per CTA, so what counts is how soon the bytes are
// asked for, not how fast they stream.
//  * The key tiles (16 keys) of a sequence are spread over the CTAs of a cluster (grid.z) and,
//    inside a CTA, over its four warps; a warp loads and processes its tiles on its own
//    (private ring of three tiles in shared memory, no CTA barrier in the loop).
//  * Keys and values of earlier positions were written by earlier steps, and the page table and
//    lengths by the host: they do not depend on the kernel before this one.  So the page ids of
//    the CTA's range are fetched, and the first tiles of every warp are requested, BEFORE the
//    kernel waits for its predecessor (programmatic dependent launch); only the query and the
//    tile that holds the newest position wait.  With 8 CTAs a context of 1,500 keys is in flight
//    before the previous kernel has ended.
//  * Partials merge in two levels: the four warps of a CTA through its own shared memory, then
//    the CTAs of the cluster through distributed shared memory with all remote reads of a row
//    issued at once.
constexpr int DK = 16;       // keys per warp tile
constexpr int DSTAGES = 3;   // tiles in flight per warp
constexpr int DEC_MAXP = 256;  // page ids of the CTA's range kept in shared memory
constexpr int DEC_Q_BYTES = 16 * ROW_BYTES;
constexpr int DEC_TILE_BYTES = DK * ROW_BYTES;
constexpr int DEC_PART_BYTES = (16 * D + 32) * 4;  // a partial: [16][D] outputs and [16][2] (m, l)
// a warp's partial after its key loop: rows 8 floats further apart than D, so that the eight rows a
// warp stores at once fall into different banks
constexpr int DEC_WPART_STRIDE = D + 8;
constexpr int DEC_WPART_BYTES = (16 * DEC_WPART_STRIDE + 32) * 4;
constexpr int DEC_RING_BYTES = DSTAGES * 2 * DEC_TILE_BYTES;
constexpr int DEC_WARP_BYTES = DEC_RING_BYTES > DEC_WPART_BYTES ? DEC_RING_BYTES : DEC_WPART_BYTES;
constexpr int DEC_CS_BYTES = D * 4;  // cos and sin of the token's angles (fused rotation)
constexpr int DEC_SMEM = DEC_Q_BYTES + 4 * DEC_WARP_BYTES + DEC_PART_BYTES + DEC_MAXP * 4 + DEC_CS_BYTES;

__device__ __forceinline__ void st_shared16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// eight elements of the low half with the eight of the high half: lo' = lo cos - hi sin, hi' = hi cos + lo sin,
// in 32-bit, rounded once (as the separate rotation kernel does)
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float* c, const float* sn) {
  bf16* a = reinterpret_cast<bf16*>(&lo);
  bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float av = __bfloat162float(a[k]), bv = __bfloat162float(b[k]);
    a[k] = __float2bfloat16(av * c[k] - bv * sn[k]);
    b[k] = __float2bfloat16(bv * c[k] + av * sn[k]);
  }
}

// four scaled outputs as bfloat16 in one 8-byte store
__device__ __forceinline__ void store_bf16x4(bf16* dst, const float4 v, const float scale) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale, v.y * scale);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale, v.w * scale);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}

// Registers are held down where the head size allows it: a CTA of this kernel shares its SM with
// the early CTAs of the product after it (and with the last ones of the product before), and that
// overlap is worth more than the registers (measured at batch 8 and 16: 238 registers, 7 % and
// 10 % slower steps than 167).
constexpr int DEC_MIN_CTAS = D <= 128 ? 3 : 1;
__global__ void __launch_bounds__(THREADS, DEC_MIN_CTAS) attn_decode_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  if (threadIdx.x == 0) ASTAMP(0);  // entry
  const uint32_t s_base = (uint32_t)__cvta_generic_to_shared(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g4 = lane >> 2, c4 = lane & 3;
  // A row's keys are cut into num_outer ranges, each range into the nsplit CTAs of one cluster.
  // The cluster merges on chip; with more than one range its result is a partial in global
  // memory and dsp_attn_combine merges the ranges.
  const int tile = blockIdx.x % p.num_dec_tiles, outer = blockIdx.x / p.num_dec_tiles;
  const int kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const bool to_partials = p.num_outer > 1;
  // the tile list, lengths and page tables come from the host, not from the kernel before
  const int seq = p.tile_seq[tile];
  const int qs = p.q_start[seq];
  const int ctx = p.ctx_len[seq];
  const int G = p.G;
  if (ctx <= 0) {  // a padding row: the whole cluster leaves (its partials say "no key seen")
    if (to_partials && split == 0 && tid < G) {
      pdl_wait();
      const size_t idx = ((size_t)qs * p.H + kvh * G + tid) * p.num_outer + outer;
      p.part_ml[idx * 2] = -INFINITY;
      p.part_ml[idx * 2 + 1] = 0.f;
    }
    return;
  }
  const int pos = ctx - 1;
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int kt_begin = lo / DK, kt_end = pos / DK + 1;
  const int per = (kt_end - kt_begin + nsplit * p.num_outer - 1) / (nsplit * p.num_outer);
  const int my_begin = kt_begin + (outer * nsplit + split) * per;
  const int my_end = min(kt_end, my_begin + per);
  const int* table = p.page_table + (size_t)seq * p.pt_stride;
  const uint32_t q_s = s_base;
  unsigned char* warp_mem = smem + DEC_Q_BYTES + warp * DEC_WARP_BYTES;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(warp_mem);
  float* cta_part = reinterpret_cast<float*>(smem + DEC_Q_BYTES + 4 * DEC_WARP_BYTES);
  int* pages_s = reinterpret_cast<int*>(smem + DEC_Q_BYTES + 4 * DEC_WARP_BYTES + DEC_PART_BYTES);
  float* cs = reinterpret_cast<float*>(smem + DEC_Q_BYTES + 4 * DEC_WARP_BYTES + DEC_PART_BYTES + DEC_MAXP * 4);
  // with the fused rotation the newest key and value are not in the cache yet: this kernel puts them there
  const bool own_new = p.fused_rope && p.write_kv;
  const int last_cached = own_new ? pos - 1 : pos;

  // ---- before the wait: page ids of this CTA's keys, then the first tiles of every warp
  const int first_page = my_begin < my_end ? (my_begin * DK) / p.page_size : 0;
  const int last_page = my_begin < my_end ? min(pos, my_end * DK - 1) / p.page_size : -1;
  const int n_pages = last_page - first_page + 1;
  const bool cached = n_pages <= DEC_MAXP;
  if (cached)
    for (int i = tid; i < n_pages; i += THREADS) pages_s[i] = table[first_page + i];
  // The cluster's merge in one level (when the rows fit the inbox): every CTA sends the rows of its
  // partial to the CTA that finishes them (row r to rank r % nsplit) by remote stores that count
  // their bytes on a barrier of the receiver; a CTA waits for the bytes due in its own inbox and
  // leaves.  No CTA reads another's memory and there is no cluster barrier after the keys.
  __shared__ __align__(8) uint64_t inbox_bar;
  const int rows_own_max = (G + nsplit - 1) / nsplit;
  const bool push_merge = nsplit > 1 && nsplit * rows_own_max <= 16;
  if (push_merge && tid == 0) {
    tc::mbar_init(&inbox_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // first half of a start barrier: by the time rows are sent, every CTA of the cluster is running
  if (push_merge) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  // a tile lies within one page when the page size is a multiple of the tile (the usual case): one
  // page lookup per tile, and a lane's pieces differ by a constant row stride
  const bool tile_in_page = p.page_size % DK == 0;
  // Tiles of this warp (bit n: its n-th tile, the first 32) that touch a page id outside the pool:
  // recorded when the tile is requested, and the whole tile of 16 keys is hidden from the softmax
  // (its rows were zero-filled, not loaded).  Nothing of this is in the loops over keys.
  uint32_t bad_tiles = 0u;
  const uint64_t once = tc::l2_policy_evict_first();
  auto load_tile = [&](int kt, int stage) {  // by one warp: consecutive lanes take consecutive 16-byte pieces of a row
    const uint32_t k_s = ring + stage * 2 * DEC_TILE_BYTES, v_s = k_s + DEC_TILE_BYTES;
    const int nth = (kt - (my_begin + warp)) >> 2;
    if (tile_in_page) {
      const int b0 = kt * DK;
      const int lp = b0 / p.page_size;
      const int page = cached ? pages_s[lp - first_page] : table[lp];
      const bool page_ok = page >= 0 && page < p.num_pages;
      if (!page_ok && b0 <= pos && b0 + DK > lo) {  // the same for every lane
        if (lane == 0) atomicOr(p.err, DSP_ERR_BAD_PAGE);
        if (nth < 32) bad_tiles |= 1u << nth;
      }
      const size_t base = (((size_t)(page_ok ? page : 0) * p.KVH + kvh) * p.page_size + (b0 % p.page_size)) * D;
      constexpr int ROWS_PER_PASS = 32 / CHUNKS > 0 ? 32 / CHUNKS : 1;
      if constexpr (32 % CHUNKS == 0) {  // whole rows per pass of the warp
        const int r0 = lane / CHUNKS, chunk = lane % CHUNKS;
#pragma unroll
        for (int r = r0; r < DK; r += ROWS_PER_PASS) {
          const int b = b0 + r;
          const bool valid = page_ok && b <= last_cached && b >= lo;
          const size_t off = base + (size_t)r * D + chunk * 8;
          cp_async16_once(k_s + sw(r, chunk), p.k_pool + (valid ? off : 0), valid, once);
          cp_async16_once(v_s + sw(r, chunk), p.v_pool + (valid ? off : 0), valid, once);
        }
      } else {
#pragma unroll 4
        for (int i = lane; i < DK * CHUNKS; i += 32) {
          const int r = i / CHUNKS, chunk = i % CHUNKS;
          const int b = b0 + r;
          const bool valid = page_ok && b <= last_cached && b >= lo;
          const size_t off = base + (size_t)r * D + chunk * 8;
          cp_async16_once(k_s + sw(r, chunk), p.k_pool + (valid ? off : 0), valid, once);
          cp_async16_once(v_s + sw(r, chunk), p.v_pool + (valid ? off : 0), valid, once);
        }
      }
      return;
    }
    bool met_bad = false;
#pragma unroll 4
    for (int i = lane; i < DK * CHUNKS; i += 32) {
      const int r = i / CHUNKS, chunk = i % CHUNKS;
      const int b = kt * DK + r;
      bool valid = b <= last_cached && b >= lo;
      size_t off = 0;
      if (valid) {
        const int lp = p.page_shift >= 0 ? (b >> p.page_shift) : (b / p.page_size);
        const int within = p.page_shift >= 0 ? (b & (p.page_size - 1)) : (b % p.page_size);
        const int page = cached ? pages_s[lp - first_page] : table[lp];
        if (page < 0 || page >= p.num_pages) {
          if (chunk == 0) atomicOr(p.err, DSP_ERR_BAD_PAGE);
          met_bad = true;
          valid = false;
        } else {
          off = (((size_t)page * p.KVH + kvh) * p.page_size + within) * D + chunk * 8;
        }
      }
      cp_async16_once(k_s + sw(r, chunk), p.k_pool + off, valid, once);
      cp_async16_once(v_s + sw(r, chunk), p.v_pool + off, valid, once);
    }
    if (__any_sync(0xffffffffu, met_bad) && nth < 32) bad_tiles |= 1u << nth;
  };

  // this warp's tiles: my_begin + warp, + 4, ...; the tile that holds the newest position (always the
  // last tile of the sequence) is requested after the wait when an earlier kernel of this step stored
  // that position, every other one may go at once
  const int first = my_begin + warp;
  const int newest = pos / DK;
  int issued = 0;  // tiles of this warp requested so far (one commit group each, in order)
  // (when this kernel stores the newest key and value itself, the tile's other rows are old as well)
  for (int j = 0; j < DSTAGES; ++j) {
    const int kt = first + 4 * j;
    if (kt >= my_end || (kt == newest && !own_new)) break;
    load_tile(kt, j);
    cp_async_commit();
    ++issued;
  }
  const int half = p.rotary_dim / 2;
  if (p.fused_rope) {
    // cos and sin of this position's angles, once for q and for the new key: they depend on the
    // position alone, so they are ready before the predecessor is
    for (int i = tid; i < half; i += THREADS) {
      float sn, c;
      sincosf((float)pos * p.inv_freq[i], &sn, &c);
      cs[i] = c;
      cs[half + i] = sn;
    }
    __syncthreads();
  }

  if (tid == 0) ASTAMP(1);  // page ids and the first tiles are requested
  pdl_wait();
  if (tid == 0) ASTAMP(2);  // the predecessor is complete
  // the next kernel (the output projection) may start now and not earlier: its weight ring would
  // compete with the key tiles requested above (measured: 1.314 ms -> 1.294 ms per decode step)
  pdl_launch_dependents();
  if (p.fused_rope) {
    // Q: the G heads of this KV head, rotated on the way into shared memory (16-byte pieces; piece j
    // of the low half rotates with piece j of the high half)
    const int hv = half / 8, tail = (D - p.rotary_dim) / 8;
    const bf16* q0 = p.q + (size_t)qs * p.q_stride + (size_t)kvh * G * D;
    for (int i = tid; i < 16 * (hv + tail); i += THREADS) {
      const int r = i / (hv + tail), j = i % (hv + tail);
      const bool valid = r < G;
      if (j < hv) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (valid) {
          lo = *reinterpret_cast<const uint4*>(q0 + (size_t)r * D + j * 8);
          hi = *reinterpret_cast<const uint4*>(q0 + (size_t)r * D + half + j * 8);
          rotate8(lo, hi, cs + j * 8, cs + half + j * 8);
        }
        st_shared16(q_s + sw(r, j), lo);
        st_shared16(q_s + sw(r, hv + j), hi);
      } else {
        const int chunk = 2 * hv + (j - hv);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (valid) v = *reinterpret_cast<const uint4*>(q0 + (size_t)r * D + chunk * 8);
        st_shared16(q_s + sw(r, chunk), v);
      }
    }
  } else {
    // Q: the G heads of this KV head, one row each
    for (int i = tid; i < 16 * CHUNKS; i += THREADS) {
      const int r = i / CHUNKS, chunk = i % CHUNKS;
      const bool valid = r < G;
      const bf16* src = valid ? p.q + (size_t)qs * p.q_stride + (size_t)(kvh * G + r) * D + chunk * 8 : p.q;
      cp_async16(q_s + sw(r, chunk), src, valid);
    }
  }
  cp_async_commit();  // every thread: one more group (Q), after its tiles
  // the ring's remaining slots, now including the newest tile
  for (int j = issued; j < DSTAGES; ++j) {
    const int kt = first + 4 * j;
    if (kt >= my_end) break;
    load_tile(kt, j);
    cp_async_commit();
    ++issued;
  }
  cp_async_wait<0>();
  __syncthreads();  // Q is complete for every warp (and this warp's first tiles with it)
  if (tid == 0) ASTAMP(3);  // Q and the first tiles have landed

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const bool row_ok[2] = {g4 < G, g4 + 8 < G};
  const int m8 = lane >> 3, l8 = lane & 7;
  // the A fragments of Q do not change over the tiles
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) ldmatrix_x4(qa[kk], q_s + sw((m8 & 1) * 8 + l8, kk * 2 + (m8 >> 1)));

  int n = 0;  // tiles of this warp done so far
  for (int kt = first; kt < my_end; kt += 4, ++n) {
    const int stage = n % DSTAGES;
    if (n >= DSTAGES) {
      // tiles beyond the first ring: the groups complete in order, at most DSTAGES - 1 may stay open
      const int ahead = issued - n - 1;  // groups requested after this tile's
      if (ahead >= 2) cp_async_wait<2>();
      else if (ahead == 1) cp_async_wait<1>();
      else cp_async_wait<0>();
      __syncwarp();
    }
    const uint32_t k_s = ring + stage * 2 * DEC_TILE_BYTES, v_s = k_s + DEC_TILE_BYTES;
    if (own_new && kt == newest) {
      // the token's own key (rotated) and value: from the fused q/k/v row into this tile and into the cache
      const int r = pos - kt * DK;
      const int hv = half / 8, tail = (D - p.rotary_dim) / 8;
      const bf16* k0 = p.q + (size_t)qs * p.q_stride + (size_t)(p.H + kvh) * D;
      const bf16* v0 = p.q + (size_t)qs * p.q_stride + (size_t)(p.H + p.KVH + kvh) * D;
      const int lp = pos / p.page_size;
      const int page = cached ? pages_s[lp - first_page] : table[lp];
      const bool page_ok = page >= 0 && page < p.num_pages;
      if (!page_ok) {  // not stored, and hidden with its tile
        if (lane == 0) atomicOr(p.err, DSP_ERR_BAD_PAGE);
        if (n < 32) bad_tiles |= 1u << n;
      }
      const size_t dst = (((size_t)(page_ok ? page : 0) * p.KVH + kvh) * p.page_size + pos % p.page_size) * D;
      bf16* k_out = const_cast<bf16*>(p.k_pool) + dst;
      bf16* v_out = const_cast<bf16*>(p.v_pool) + dst;
      for (int i = lane; i < hv + tail + CHUNKS; i += 32) {
        if (i < hv) {
          uint4 klo = *reinterpret_cast<const uint4*>(k0 + i * 8);
          uint4 khi = *reinterpret_cast<const uint4*>(k0 + half + i * 8);
          rotate8(klo, khi, cs + i * 8, cs + half + i * 8);
          st_shared16(k_s + sw(r, i), klo);
          st_shared16(k_s + sw(r, hv + i), khi);
          if (page_ok) {
            *reinterpret_cast<uint4*>(k_out + i * 8) = klo;
            *reinterpret_cast<uint4*>(k_out + half + i * 8) = khi;
          }
        } else if (i < hv + tail) {
          const int chunk = 2 * hv + (i - hv);
          const uint4 kv = *reinterpret_cast<const uint4*>(k0 + chunk * 8);
          st_shared16(k_s + sw(r, chunk), kv);
          if (page_ok) *reinterpret_cast<uint4*>(k_out + chunk * 8) = kv;
        } else {
          const int chunk = i - hv - tail;
          const uint4 vv = *reinterpret_cast<const uint4*>(v0 + chunk * 8);
          st_shared16(v_s + sw(r, chunk), vv);
          if (page_ok) *reinterpret_cast<uint4*>(v_out + chunk * 8) = vv;
        }
      }
      __syncwarp();
    }
    float s[DK / 8][4];
#pragma unroll
    for (int i = 0; i < DK / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b[4];
      ldmatrix_x4(b, k_s + sw((m8 >> 1) * 8 + l8, kk * 2 + (m8 & 1)));
      mma_bf16(s[0], qa[kk], b[0], b[1]);
      mma_bf16(s[1], qa[kk], b[2], b[3]);
    }
    const int pos_t = (n < 32 && ((bad_tiles >> n) & 1u)) ? -1 : pos;  // no key of such a tile is visible
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int key = kt * DK + nt * 8 + 2 * c4 + (e & 1);
        const bool vis = row_ok[r] && key <= pos_t && key >= lo;
        const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = v;
        tmax[r] = fmaxf(tmax[r], v);
      }
    float alpha[2], m_safe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      const float m_new = fmaxf(m_run[r], tmax[r]);
      m_safe[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_safe[r]);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nt][e] - m_safe[e >> 1]);
        s[nt][e] = pv;
        l_run[e >> 1] += pv;
      }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
    {
      uint32_t a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int dd = 0; dd < D / 16; ++dd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_s + sw((m8 & 1) * 8 + l8, dd * 2 + (m8 >> 1)));
        mma_bf16(o[2 * dd], a, b[0], b[1]);
        mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
      }
    }
    // the slot is free: the tile DSTAGES further on goes into it
    const int next = kt + 4 * DSTAGES;
    if (next < my_end) {
      __syncwarp();
      load_tile(next, stage);
      cp_async_commit();
      ++issued;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (tid == 0) ASTAMP(4);  // warp 0 is through its key tiles
  // ---- level 1: the warp's partial into its own (now free) ring memory, merged over the CTA's warps
  __syncwarp();
  {
    float* part_o = reinterpret_cast<float*>(warp_mem);
    float* part_ml = part_o + 16 * DEC_WPART_STRIDE;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g4 + 8 * r;
      if (row >= G) continue;  // rows beyond the group are never read
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(part_o + row * DEC_WPART_STRIDE + i * 8 + 2 * c4) =
            make_float2(o[i][2 * r], o[i][2 * r + 1]);
      if (c4 == 0) {
        part_ml[row * 2] = m_run[r];
        part_ml[row * 2 + 1] = l_run[r];
      }
    }
  }
  __syncthreads();
  if (tid == 0) ASTAMP(5);  // every warp of the CTA is through
  if (push_merge) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // second half
  if (tid == 0) ASTAMP(10);  // the cluster's CTAs are all running
  const bool last_level = nsplit == 1;
  // The merges run once per CTA and their cost is latency: dependent instructions, and transactions
  // between CTAs.  So a thread owns four consecutive outputs of one row, asks for all partials of
  // them at once and weighs them itself (every thread of a row repeats the few exponentials: no
  // exchange between lanes), and a row leaves in one 16-byte store per thread.
  constexpr int C4 = D / 4;  // 16-byte pieces of an output row
  for (int item = tid; item < G * C4; item += THREADS) {
    const int row = item / C4, c = item - row * C4;
    float2 ml[4];
    float4 v[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* part = reinterpret_cast<const float*>(smem + DEC_Q_BYTES + w * DEC_WARP_BYTES);
      ml[w] = *reinterpret_cast<const float2*>(part + 16 * DEC_WPART_STRIDE + row * 2);
      v[w] = *reinterpret_cast<const float4*>(part + row * DEC_WPART_STRIDE + c * 4);
    }
    const float M = fmaxf(fmaxf(ml[0].x, ml[1].x), fmaxf(ml[2].x, ml[3].x));
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = ml[w].x == -INFINITY ? 0.f : exp2f(ml[w].x - M);
      L += wgt * ml[w].y;
      acc.x += wgt * v[w].x, acc.y += wgt * v[w].y, acc.z += wgt * v[w].z, acc.w += wgt * v[w].w;
    }
    if (last_level && to_partials) {
      const size_t idx = ((size_t)qs * p.H + kvh * G + row) * p.num_outer + outer;
      reinterpret_cast<float4*>(p.part_o + idx * D)[c] = acc;
      if (c == 0) *reinterpret_cast<float2*>(p.part_ml + idx * 2) = make_float2(M, L);
    } else if (last_level) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      store_bf16x4(p.out + (size_t)qs * p.out_stride + (size_t)(kvh * G + row) * D + 4 * c, acc, inv);
    } else if (push_merge) {
      // slot (this rank, the row's place among its owner's rows) of the owner's inbox
      const uint32_t owner = (uint32_t)(row % nsplit);
      const int q = split * rows_own_max + row / nsplit;
      const uint32_t bar = tc::mapa_u32(tc::smem_u32(&inbox_bar), owner);
      tc::st_async_v4(tc::mapa_u32(tc::smem_u32(cta_part + q * D + c * 4), owner), acc, bar);
      if (c == 0)
        tc::st_async_v2(tc::mapa_u32(tc::smem_u32(cta_part + 16 * D + q * 2), owner), make_float2(M, L), bar);
    } else {
      reinterpret_cast<float4*>(cta_part + row * D)[c] = acc;
      if (c == 0) {
        cta_part[16 * D + row * 2] = M;
        cta_part[16 * D + row * 2 + 1] = L;
      }
    }
  }
  if (tid == 0) ASTAMP(8);  // this CTA's rows are merged
  if (last_level) return;
  if (push_merge) {
    // the rows this CTA finishes: split, split + nsplit, ...; every rank sends D + 2 floats of each
    if (tid == 0) ASTAMP(6);  // this CTA's rows are on their way
    const int rows_own = split < G ? (G - split + nsplit - 1) / nsplit : 0;
    if (tid == 0) tc::mbar_expect_tx(&inbox_bar, (uint32_t)(nsplit * rows_own * (D + 2) * 4));
    if (!tc::mbar_wait(&inbox_bar, 0)) {
      if (tid == 0) atomicOr(p.err, DSP_ERR_WAIT_LIMIT);
      return;
    }
    if (tid == 0) ASTAMP(7);  // every rank's rows have arrived
    for (int item = tid; item < rows_own * C4; item += THREADS) {
      const int slot = item / C4, c = item - slot * C4;
      const int row = split + slot * nsplit;
      float2 ml[8];
      float4 v[8];
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < 8; ++r) {  // the decode kernel runs with at most 8 splits
        const int q = (r < nsplit ? r : 0) * rows_own_max + slot;
        ml[r] = *reinterpret_cast<const float2*>(cta_part + 16 * D + q * 2);
        v[r] = *reinterpret_cast<const float4*>(cta_part + q * D + c * 4);
        if (r >= nsplit) ml[r].x = -INFINITY;
        M = fmaxf(M, ml[r].x);
      }
      float L = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float wgt = ml[r].x == -INFINITY ? 0.f : exp2f(ml[r].x - M);
        L += wgt * ml[r].y;
        acc.x += wgt * v[r].x, acc.y += wgt * v[r].y, acc.z += wgt * v[r].z, acc.w += wgt * v[r].w;
      }
      if (to_partials) {
        const size_t idx = ((size_t)qs * p.H + kvh * G + row) * p.num_outer + outer;
        reinterpret_cast<float4*>(p.part_o + idx * D)[c] = acc;
        if (c == 0) *reinterpret_cast<float2*>(p.part_ml + idx * 2) = make_float2(M, L);
      } else {
        const float inv = L > 0.f ? 1.f / L : 0.f;
        store_bf16x4(p.out + (size_t)qs * p.out_stride + (size_t)(kvh * G + row) * D + 4 * c, acc, inv);
      }
    }
    if (tid == 0) ASTAMP(9);  // end
    return;
  }
  // ---- level 2: the CTAs of the cluster; the rows are dealt to its warps
  if (tid == 0) ASTAMP(6);  // the CTA's partial is in its shared memory
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  if (tid == 0) ASTAMP(7);  // every CTA of the cluster is there
  for (int row = split * 4 + warp; row < G; row += nsplit * 4) {
    float m_c[8], l_c[8];
    const float* remote[8];
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      remote[c] = cluster.map_shared_rank(cta_part, c < nsplit ? c : 0);
      m_c[c] = c < nsplit ? remote[c][16 * D + row * 2] : -INFINITY;
      l_c[c] = c < nsplit ? remote[c][16 * D + row * 2 + 1] : 0.f;
    }
    // all partial outputs of the row are requested before any is used
    float po[8][(D + 31) / 32];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int j = 0; j < (D + 31) / 32; ++j) {
        const int d = lane + 32 * j;
        po[c][j] = (c < nsplit && d < D) ? remote[c][row * D + d] : 0.f;
      }
#pragma unroll
    for (int c = 0; c < 8; ++c) M = fmaxf(M, m_c[c]);
    float L = 0.f;
    float acc[(D + 31) / 32];
#pragma unroll
    for (int j = 0; j < (D + 31) / 32; ++j) acc[j] = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float wgt = m_c[c] == -INFINITY ? 0.f : exp2f(m_c[c] - M);
      L += wgt * l_c[c];
#pragma unroll
      for (int j = 0; j < (D + 31) / 32; ++j) acc[j] += wgt * po[c][j];
    }
    if (to_partials) {
      const size_t idx = ((size_t)qs * p.H + kvh * G + row) * p.num_outer + outer;
#pragma unroll
      for (int j = 0; j < (D + 31) / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < D) p.part_o[idx * D + d] = acc[j];
      }
      if (lane == 0) {
        p.part_ml[idx * 2] = M;
        p.part_ml[idx * 2 + 1] = L;
      }
      continue;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    bf16* dst = p.out + (size_t)qs * p.out_stride + (size_t)(kvh * G + row) * D;
#pragma unroll
    for (int j = 0; j < (D + 31) / 32; ++j) {
      const int d = lane + 32 * j;
      if (d < D) dst[d] = __float2bfloat16(acc[j] * inv);
    }
  }
  if (tid == 0) ASTAMP(8);  // this CTA's rows are stored
  cluster.sync();  // nobody leaves while its partials may still be read
  if (tid == 0) ASTAMP(9);  // end
}
}  // namespace

#ifdef DSP_STAMPS
namespace {
long g_astamp_cursor = -1;
long g_astamp_log[4096][2];
int g_astamp_launches = 0;
}  // namespace
extern "C" long DSP_CAT(dsp_attn_stamps_control_d, DSP_HEAD_DIM)(int on) {
  const long used = g_astamp_cursor < 0 ? 0 : g_astamp_cursor;
  g_astamp_cursor = on ? 0 : -1;
  if (on) g_astamp_launches = 0;
  return used;
}
extern "C" int DSP_CAT(dsp_attn_stamps_log_d, DSP_HEAD_DIM)(long* out, int max_launches) {
  const int n = g_astamp_launches < max_launches ? g_astamp_launches : max_launches;
  for (int i = 0; i < n; ++i) {
    out[i * 2] = g_astamp_log[i][0];
    out[i * 2 + 1] = g_astamp_log[i][1];
  }
  return n;
}
extern "C" int DSP_CAT(dsp_attn_stamps_read_d, DSP_HEAD_DIM)(unsigned long long* out, long n) {
  return cudaMemcpyFromSymbol(out, g_attn_stamps, (size_t)n * sizeof(unsigned long long)) == cudaSuccess ? 0 : 1;
}
#endif

// Runs tiles [tile_offset, tile_offset + num_tiles) of the tile list.  With num_splits > 1 and no
// cluster the partials go to part_o / part_ml, [row][num_splits], and dsp_attn_combine must follow.
// The single-token kernel (decode_only) takes num_outer key ranges per row on top of the cluster's
// num_splits; with num_outer > 1 its partials are [row][num_outer] and dsp_attn_combine follows.
extern "C" int DSP_CAT(dsp_attn_mma_d, DSP_HEAD_DIM)(
    const void* q, long q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int pt_stride, const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_tok0,
    int tile_offset, int num_tiles, void* out, long out_stride, float* part_o, float* part_ml, int H,
    int KVH, int tokens_per_tile, int page_size, int num_pages, int window, int num_splits,
    int cluster_combine, int decode_only, int num_outer, float scale, const float* inv_freq, int rotary_dim, int fused_rope,
    int write_kv, int* err, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (KVH <= 0 || H % KVH != 0 || (H / KVH) * tokens_per_tile > BM || tokens_per_tile < 1) return 2;
  if (num_splits < 1 || num_splits > 65535 || KVH > 65535) return 2;
  if (num_splits > 1 && !cluster_combine && (part_o == nullptr || part_ml == nullptr)) return 2;
  if (cluster_combine && !decode_only && (num_splits < 2 || num_splits > 8)) return 2;
  if (num_outer < 1 || (num_outer > 1 && (!decode_only || part_o == nullptr || part_ml == nullptr))) return 2;
  if ((long)num_tiles * num_outer > 0x7fffffffL) return 2;
  if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q % 16) || ((uintptr_t)k_pool % 16) ||
      ((uintptr_t)v_pool % 16) || ((uintptr_t)out % 4))
    return 3;
  Params p;
  p.q = (const bf16*)q;
  p.q_stride = q_stride;
  p.k_pool = (const bf16*)k_pool;
  p.v_pool = (const bf16*)v_pool;
  p.page_table = page_table;
  p.pt_stride = pt_stride;
  p.q_start = q_start;
  p.ctx_len = ctx_len;
  p.tile_seq = tile_seq;
  p.tile_tok0 = tile_tok0;
  p.out = (bf16*)out;
  p.out_stride = out_stride;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.H = H;
  p.KVH = KVH;
  p.G = H / KVH;
  p.tokens_per_tile = tokens_per_tile;
  p.page_size = page_size;
  p.page_shift = (page_size > 0 && (page_size & (page_size - 1)) == 0) ? __builtin_ctz(page_size) : -1;
  p.num_pages = num_pages;
  p.window = window;
  p.num_splits = num_splits;
  p.cluster_combine = cluster_combine;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = err;
  p.inv_freq = inv_freq;
  p.rotary_dim = rotary_dim;
  p.fused_rope = fused_rope;
  p.write_kv = write_kv;
  p.num_outer = num_outer;
  p.num_dec_tiles = num_tiles;
  if (fused_rope) {
    // only the single-token kernel rotates, and in 16-byte pieces
    if (!(decode_only && p.G <= 16 && num_splits <= 8 && DEC_SMEM <= 227 * 1024)) return 2;
    if (inv_freq == nullptr || rotary_dim <= 0 || rotary_dim > D || rotary_dim % 16 != 0) return 2;
  }
  const int smem = 5 * TILE_BYTES;
  static bool configured = false;  // once; not repeated under graph capture
  if (!configured) {
    if (cudaFuncSetAttribute(attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return 4;
    configured = true;
  }
  dim3 grid(num_tiles, KVH, num_splits);
  // single decoded tokens whose group fits one 16-row tile: the warp-parallel kernel
  p.stamp_base = -1;
  if (decode_only && p.G <= 16 && num_splits <= 8 && DEC_SMEM <= 227 * 1024) {
#ifdef DSP_STAMPS
    {
      const long ctas = (long)num_tiles * num_outer * KVH * num_splits;
      if (g_astamp_cursor >= 0 && g_astamp_cursor + ctas * 12 <= (1 << 20) && g_astamp_launches < 4096) {
        p.stamp_base = g_astamp_cursor;
        g_astamp_log[g_astamp_launches][0] = g_astamp_cursor;
        g_astamp_log[g_astamp_launches][1] = ctas;
        ++g_astamp_launches;
        g_astamp_cursor += ctas * 12;
      }
    }
#endif
    static bool dec_configured = false;
    if (!dec_configured) {
      if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM) != cudaSuccess)
        return 4;
      dec_configured = true;
    }
    if (tile_offset != 0) return 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_tiles * num_outer, KVH, num_splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)DEC_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = num_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    prefer_max_shared(reinterpret_cast<const void*>(attn_decode_kernel));
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel, p) == cudaSuccess ? 0 : 1;
  }
  if (num_outer > 1) return 2;  // only the single-token kernel cuts a row's keys beyond the cluster
  if (cluster_combine) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = num_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    prefer_max_shared(reinterpret_cast<const void*>(attn_mma_kernel));
    return cudaLaunchKernelEx(&cfg, attn_mma_kernel, p, tile_offset) == cudaSuccess ? 0 : 1;
  }
  return launch_pdl(attn_mma_kernel, grid, dim3(THREADS), (size_t)smem, stream, p, tile_offset) == cudaSuccess ? 0 : 1;
}
