// Causal grouped-query attention for portions of prompts on the fifth-generation tensor cores:
// S = Q K^T and O += P V are tcgen05.mma with the accumulators and the A operands (Q, P) in tensor
// memory, keys and values come from the paged cache by TMA (one request per page, or one per
// operand and tile where the tile's pages follow one another in the pool), bfloat16 in, 32-bit
// softmax and accumulation.  Compiled once per head size (-DDSP_HEAD_DIM=64 or 128).
//
// A tile is 128 query rows of one KV head of one sequence; a row is a (token, head-in-group)
// pair, so the G query heads that share a KV head share every key/value load.  Keys are walked in
// tiles of 64 through the page table.  Roles, one CTA per tile:
//   warp 0      issues the TMA loads of the K tiles and of the V tiles, each into a ring of its own: a
//               K tile is free again when its scores are complete, a V tile two softmax iterations
//               later, when its output product is;
//   warps 1, 11 one thread each issues the score products S[i] = Q K[i]^T of one softmax group;
//   warp 10     one thread issues the output products O[i % 2] += P[i] V[i];
//   warps 2..9  two softmax groups of four warps.  Group g owns the key tiles i = g, g + 2, ...: its own
//               score buffer S[g], output accumulator O[g] and P[g] in tensor memory and its own
//               running maximum and sum, so the two groups never exchange anything until the end
//               and the softmax of tile i + 1 runs beside that of tile i.  In a group thread r owns
//               row r (lane r of tensor memory): it reads its 64 scores, rescales its row of O[g]
//               when the running maximum moved by more than 2^8, and writes P as bfloat16, two per
//               column.  At the end group 0 merges the two partial results (like two key splits)
//               and stores the rows.
// The query at position p sees keys b with max(0, p - window + 1) <= b <= p.  Value rows of keys
// that no row of the tile may see (beyond the last position, before the window, on pages that were
// given back) are zeroed in shared memory before the second product, so stale cache contents never
// reach the tensor cores as 0 * x.  Every wait on a barrier is bounded; a wait that runs out sets
// the device error word and the CTA returns after freeing its tensor memory.
#include "tcgen05_common.cuh"

#ifndef DSP_HEAD_DIM
#error "compile with -DDSP_HEAD_DIM=<head size>"
#endif

#define DSP_CAT2(a, b) a##b
#define DSP_CAT(a, b) DSP_CAT2(a, b)

namespace {
using namespace tc;

constexpr int D = DSP_HEAD_DIM;
static_assert(D == 64 || D == 128, "this kernel is built for head sizes 64 and 128");
constexpr int BM = 128, BN = 64, THREADS = 384;
constexpr int K_STAGES = 5, V_STAGES = 7;  // tiles in the ring of keys and in the ring of values
constexpr int BAD_SLOTS = 16;              // a tile's unreadable pages are remembered until its softmax has begun
static_assert(BAD_SLOTS >= K_STAGES + 4, "a slot is rewritten K_STAGES + 4 tiles later at the earliest");
// warp 0: TMA, warps 1 and 11: issue S = Q K^T for softmax group 0 and 1, warps 2-9: softmax, warp 10: issues O += P V
constexpr int PV_WARP = 10, S1_WARP = 11;
constexpr int KD = D / 64;            // 64-wide slices of the head dimension (128-byte rows)
constexpr int KV_SLICE = BN * 128;    // bytes of one slice of a K or V tile
constexpr int KV_BYTES = KD * KV_SLICE;
constexpr int SMEM_BYTES = (K_STAGES + V_STAGES) * KV_BYTES + 1024;
static_assert(SMEM_BYTES + 1536 <= 227 * 1024, "dynamic and static shared memory of a CTA");
// Tensor memory, 32-bit columns: two score buffers, two output accumulators, and the A operands of
// both products, two bfloat16 per column: P of each group (64 keys) and the Q tile.  Operands that
// the tensor cores take from tensor memory cost no shared-memory bandwidth: with Q and P in shared
// memory, a key tile moved 128 KB through the shared-memory port (Q 32, K 16, P 16 written and 16
// read, V 16, the arriving tiles 32), 1,000 of the 1,200 cycles that a tile took, and every
// barrier operation of the control warps waited in that queue.
constexpr int S_COLS = BN;                 // columns of one score buffer
constexpr int O_COL = 2 * S_COLS;          // the two output accumulators follow the two score buffers
constexpr int P_COLS = BN / 2;             // columns of one group's P
constexpr int P_COL = O_COL + 2 * D;
constexpr int Q_COL = P_COL + 2 * P_COLS;  // D / 2 columns
constexpr int TMEM_COLS = 512;
static_assert(Q_COL + D / 2 <= TMEM_COLS, "tensor memory layout");
constexpr float RESCALE_STEP = 8.f;   // the running maximum follows the true one in steps of 2^8

struct Params {
  const bf16* q;
  long q_stride;
  const int* page_table;
  int pt_stride;
  const int* q_start;
  const int* ctx_len;
  const int* tile_seq;
  const int* tile_tok0;
  bf16* out;
  long out_stride;
  int H, KVH, G, tokens_per_tile, page_size, num_pages, window;
  int page_runs;  // the run maps are valid
  float scale_log2;
  int* err;
};

// value tile as the B operand of O += P V: N (head dimension) contiguous, 64 per 128-byte row,
// one row per key; slices of 64 columns lbo bytes apart, groups of 8 keys 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void st_shared16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_tcgen05_kernel(const Params p, int tile_offset, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap runs_k,
                    const __grid_constant__ CUtensorMap runs_v) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1024 bytes
  __shared__ __align__(8) uint64_t k_full[K_STAGES];   // the K tile has landed
  __shared__ __align__(8) uint64_t k_empty[K_STAGES];  // the tile's scores are complete
  __shared__ __align__(8) uint64_t v_full[V_STAGES];   // the V tile has landed
  __shared__ __align__(8) uint64_t v_empty[V_STAGES];  // the tile's output product is complete
  __shared__ __align__(8) uint64_t s_full[2];         // a score buffer is complete
  __shared__ __align__(8) uint64_t s_free[2];         // the group has read its score buffer
  __shared__ __align__(8) uint64_t p_full[2];         // P written, O rescaled, V rows zeroed
  __shared__ __align__(8) uint64_t o_done[2];         // O[g] += P V of a tile is complete
  __shared__ __align__(8) uint64_t q_ready;           // the Q tile is in tensor memory
  __shared__ float merge_m[BM], merge_l[BM];          // group 1's running maximum and sum per row
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  __shared__ uint32_t bad_pages[BAD_SLOTS];  // of key tile i, in slot i % BAD_SLOTS; bit j: page j had no valid id (not loaded)

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // later tiles of a prompt see more keys: the longest work is scheduled first
  const int tile = ((int)gridDim.x - 1 - (int)blockIdx.x) + tile_offset, kvh = blockIdx.y;
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
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;            // first key any row sees
  const int lo_top = p.window > 0 ? max(0, pos_last - p.window + 1) : 0;    // first key every row sees
  const int kt_begin = lo / BN, kt_end = pos_last / BN + 1;
  const int n_kt = kt_end - kt_begin;
  const int* table = p.page_table + (size_t)seq * p.pt_stride;

  unsigned char* k_s = smem;                                  // [stage][slice][64 keys][128 bytes]
  unsigned char* v_s = k_s + K_STAGES * KV_BYTES;

  if (tid == 0) {
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_free[b], 4);
      mbar_init(&p_full[b], 4);  // one arrival per warp of the group
      mbar_init(&o_done[b], 1);
    }
    mbar_init(&q_ready, 4);  // one arrival per warp that writes a quarter of the tile
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // ---- Q tile: thread r of warps 2..5 fetches row r (rows past the tile are zero) while the tensor
  // memory is being allocated, and writes it there afterwards: lane r, two bfloat16 per column
  uint4 q_row[D / 8];
  if (warp >= 2 && warp < 6) {
    const int r = (warp & 3) * 32 + lane;
    const bool valid = r < nrows;
    const uint4* src = nullptr;
    if (valid)
      src = reinterpret_cast<const uint4*>(p.q + (size_t)(qs + tok0 + r / G) * p.q_stride +
                                           (size_t)(kvh * G + r % G) * D);
#pragma unroll
    for (int c = 0; c < D / 8; ++c) q_row[c] = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp >= 2 && warp < 6) {
    const uint32_t q_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)Q_COL;
#pragma unroll
    for (int c0 = 0; c0 < D / 2; c0 += 32) {
      uint32_t w[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        w[4 * c] = q_row[c0 / 4 + c].x;
        w[4 * c + 1] = q_row[c0 / 4 + c].y;
        w[4 * c + 2] = q_row[c0 / 4 + c].z;
        w[4 * c + 3] = q_row[c0 / 4 + c].w;
      }
      tmem_st32(q_addr + (uint32_t)c0, w);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_ready);
  }

  if (warp == 0) {
    // ---- TMA producer of the K tiles and the V tiles, each into a ring of its own
    const int pages_per_tile = BN / p.page_size;
    const uint32_t page_bytes = (uint32_t)KD * (uint32_t)p.page_size * 128u;  // every slice, of K or of V
    // Page ids are looked up for a chunk of 32 / pages_per_tile key tiles at a time, lane l
    // holding page l % pages_per_tile of the chunk's tile l / pages_per_tile, and the chunk after
    // the current one is asked for while the current one is walked.  What a tile needs (is a page
    // wanted, has it a valid id, do the tile's pages follow one another in the pool) is worked
    // out for the whole chunk with one shuffle and three votes, and the tile's first lane, which
    // holds its first page, waits for the ring slot and issues the request: per tile the loop
    // then has one barrier operation in a row, where a table read, issued one tile ahead (900
    // cycles under load), or four shuffles (250 cycles each while the softmax warps keep the
    // shared-memory pipe busy) set the pace of the whole kernel; a tile arrives 500 cycles
    // after its request.
    const int ppt_shift = __ffs(pages_per_tile) - 1;  // page sizes are powers of two here
    const int page_shift_p = __ffs(p.page_size) - 1;
    const int chunk_shift = 5 - ppt_shift, chunk_mask = (1 << chunk_shift) - 1;  // tiles per chunk
    const int page_in_tile = lane & (pages_per_tile - 1);
    const uint32_t tile_lanes = pages_per_tile == 32 ? 0xffffffffu : ((1u << pages_per_tile) - 1u);
    auto load_chunk = [&](int c) -> int {
      const int i = (c << chunk_shift) + (lane >> ppt_shift);
      const int first = (kt_begin + i) * BN + page_in_tile * p.page_size;
      if (i < n_kt && first <= pos_last && first + p.page_size > lo) return table[first >> page_shift_p];
      return -2;  // not wanted
    };
    int pg = -2, pg_next = load_chunk(0);
    uint32_t bad_mask = 0, live_mask = 0, run_mask = 0;
    // Two tiles per turn, each with a lane of its own that waits for the tile's ring slots and
    // issues its requests: the waits, the announcements and the requests of both run side by side
    // (a turn costs some 900 cycles of latencies in a row, whatever it does, and at one tile per
    // turn this warp set the kernel's pace once the products took their operands from tensor memory).
    int sk = 0, rk = 0, sv = 0, rv = 0;  // ring slots of K and of V of the turn's first tile, and their use counts
    for (int i = 0; i < n_kt; i += 2) {
      const int in_chunk = i & chunk_mask;  // chunks hold an even number of tiles
      if (in_chunk == 0) {
        pg = pg_next;
        pg_next = load_chunk((i >> chunk_shift) + 1);
        // a page id outside the pool: recorded, not loaded, and its keys are hidden from every row
        const bool bad = pg != -2 && (pg < 0 || pg >= p.num_pages);
        if (bad) {
          atomicOr(p.err, DSP_ERR_BAD_PAGE);
          pg = -1;
        }
        bad_mask = __ballot_sync(0xffffffffu, bad);
        live_mask = __ballot_sync(0xffffffffu, pg >= 0);
        const int first_pg = __shfl_sync(0xffffffffu, pg, lane & ~(pages_per_tile - 1));
        run_mask = __ballot_sync(0xffffffffu, pg >= 0 && pg == first_pg + page_in_tile &&
                                                  first_pg + pages_per_tile <= p.num_pages);
      }
      const int second = (lane >> ppt_shift) - in_chunk;  // 0, 1: this lane holds a page of the turn's first, second tile
      const bool mine = (second == 0 || second == 1) && i + second < n_kt;
      const int shift = (in_chunk + (second == 1 ? 1 : 0)) << ppt_shift;  // first lane of this lane's tile
      const uint32_t live = (live_mask >> shift) & tile_lanes;
      const bool in_run = p.page_runs && ((run_mask >> shift) & tile_lanes) == tile_lanes;
      const bool leader = mine && lane == shift;
      int my_sk = sk, my_rk = rk, my_sv = sv, my_rv = rv;
      if (second == 1) {
        if (++my_sk == K_STAGES) {
          my_sk = 0;
          ++my_rk;
        }
        if (++my_sv == V_STAGES) {
          my_sv = 0;
          ++my_rv;
        }
      }
      if (leader) {
        if (*(volatile int*)&failed == 0 &&
            mbar_wait_both(&k_empty[my_sk], (my_rk & 1) ^ 1, &v_empty[my_sv], (my_rv & 1) ^ 1)) {
          bad_pages[(i + second) % BAD_SLOTS] = (bad_mask >> shift) & tile_lanes;  // published by the arrival on k_full below
          if (live == 0) {
            mbar_arrive(&k_full[my_sk]);
            mbar_arrive(&v_full[my_sv]);
          } else {
            mbar_expect_tx(&k_full[my_sk], (uint32_t)__popc(live) * page_bytes);
            mbar_expect_tx(&v_full[my_sv], (uint32_t)__popc(live) * page_bytes);
          }
          // The tile's pages lie one after the other in the pool (what a pool hands out while it
          // is not fragmented): one request per operand brings them all, where a page of 16
          // tokens otherwise takes KD requests of 2 KB, and the requests, not the bytes, are what
          // the TMA unit's time goes to.  Both ways leave the same bytes at the same places.
          if (in_run) {
            tma_load_4d(k_s + my_sk * KV_BYTES, &runs_k, &k_full[my_sk], 0, kvh * p.page_size, pg, 0);
            tma_load_4d(v_s + my_sv * KV_BYTES, &runs_v, &v_full[my_sv], 0, kvh * p.page_size, pg, 0);
          }
        } else {
          failed = 1;  // nothing more is loaded; the warps that wait for tiles give up in their turn
        }
      }
      if (!__all_sync(0xffffffffu, !mine || in_run)) {
        // some tile of the turn goes page by page: the bytes were announced above, before any
        // lane's load can count them
        if (mine && !in_run && pg >= 0 && *(volatile int*)&failed == 0) {
          const int row = (pg * p.KVH + kvh) * p.page_size;
          const int dst = page_in_tile * p.page_size * 128;
#pragma unroll
          for (int h = 0; h < KD; ++h) {
            tma_load_2d(k_s + my_sk * KV_BYTES + dst + h * KV_SLICE, &map_k, &k_full[my_sk], h * 64, row);
            tma_load_2d(v_s + my_sv * KV_BYTES + dst + h * KV_SLICE, &map_v, &v_full[my_sv], h * 64, row);
          }
        }
      }
      for (int u = 0; u < 2; ++u) {
        if (++sk == K_STAGES) {
          sk = 0;
          ++rk;
        }
        if (++sv == V_STAGES) {
          sv = 0;
          ++rv;
        }
      }
    }
  } else if (warp == 1 || warp == S1_WARP) {
    // ---- issuers of the score products: warp 1 for the tiles of softmax group 0, warp S1_WARP for
    // those of group 1.  One thread for both spent 340 cycles per tile on barriers that were long
    // complete and 700 on issuing eight products and two commits, and these 1,250 cycles a tile,
    // in one thread, were the kernel's pace.
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(BM, BN);
      // descriptors are linear in the address: the tile's base once, a constant per k step
      const uint64_t k_desc0 = umma_desc(smem_u32(k_s));
      auto issue_scores = [&](int i) {
        const int s = i % K_STAGES;
        tc_fence_after();
        const uint64_t k_desc = k_desc0 + (uint64_t)(s * (KV_BYTES >> 4));
        const uint32_t tmem_s = tmem_base + (uint32_t)((i & 1) * S_COLS);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2), in = (uint32_t)(k & 3) * 32u;
          umma_a_tmem(tmem_s, tmem_base + (uint32_t)(Q_COL + k * 8), k_desc + ((off * KV_SLICE + in) >> 4), idesc_s, k != 0);
        }
        umma_commit(&s_full[i & 1]);
        umma_commit(&k_empty[s]);
      };
      // The scores of tile a need K[a] and, from the group's second tile on, that the group has
      // read S[a % 2] (tile a - 2).
      bool ok = mbar_wait(&q_ready, 0);
      tc_fence_after();
      for (int a = warp == 1 ? 0 : 1; a < n_kt && ok; a += 2) {
        ok = a < 2 ? mbar_wait(&k_full[a % K_STAGES], (a / K_STAGES) & 1)
                   : mbar_wait_both(&k_full[a % K_STAGES], (a / K_STAGES) & 1, &s_free[a & 1], ((a - 2) >> 1) & 1);
        if (ok) issue_scores(a);
      }
      if (!ok) failed = 1;
    }
  } else if (warp == PV_WARP) {
    // ---- issuer of the output products: O[g] += P[b] V[b] needs P[b] (written, O rescaled, dead value rows zeroed)
    if (lane == 0) {
      const uint32_t idesc_o = umma_idesc(BM, D) | (1u << 16);  // B (values) is N-major
      const uint64_t v_desc0 = umma_desc_mn(smem_u32(v_s), KV_SLICE);
      bool ok = true;
      for (int b = 0; b < n_kt && ok; ++b) {
        const int g = b & 1, st = b % V_STAGES;
        ok = mbar_wait_both(&v_full[st], (b / V_STAGES) & 1, &p_full[g], (b >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint64_t v_desc = v_desc0 + (uint64_t)(st * (KV_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          umma_a_tmem(tmem_base + (uint32_t)(O_COL + g * D), tmem_base + (uint32_t)(P_COL + g * P_COLS + k * 8),
                      v_desc + (uint64_t)(k * 128), idesc_o, (b >= 2) || k != 0);
        umma_commit(&v_empty[st]);
        umma_commit(&o_done[g]);
      }
      if (!ok) failed = 1;
    }
  } else {
    // ---- softmax groups: thread r of group g owns row r for the key tiles g, g + 2, ...
    const int g = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const bool row_ok = r < nrows;
    const int pos_r = pos0 + r / G;
    const int lo_r = p.window > 0 ? pos_r - p.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)(g * S_COLS);
    const uint32_t o_addr = lane_addr + (uint32_t)(O_COL + g * D);
    const uint32_t p_addr = lane_addr + (uint32_t)(P_COL + g * P_COLS);
    const float scale = p.scale_log2;
    const int page_shift = __ffs(p.page_size) - 1;  // page sizes are powers of two here
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int j = 0;  // tiles of this group so far
    for (int i = g; i < n_kt; i += 2, ++j) {
      const int key0 = (kt_begin + i) * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[g], j & 1))) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sv[64];
      {
        uint32_t a[32], b[32];
        tmem_ld32(s_addr, a);
        tmem_ld32(s_addr + 32, b);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          sv[c] = a[c];
          sv[32 + c] = b[c];
        }
      }
      // the scores are in registers: the next scores of this group may overwrite S[g]
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[g]);
      // tiles every row of the CTA sees whole (most of them) skip the mask
      const uint32_t bad = bad_pages[i % BAD_SLOTS];
      if (!(key0 + BN - 1 <= pos0 && key0 >= lo_top) || bad != 0u) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          const bool vis = row_ok && key <= pos_r && key >= lo_r && !((bad >> (c >> page_shift)) & 1u);
          sv[c] = vis ? sv[c] : 0xff800000u;  // -inf
        }
      }
      float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        t0 = fmaxf(t0, __uint_as_float(sv[c]));
        t1 = fmaxf(t1, __uint_as_float(sv[c + 1]));
        t2 = fmaxf(t2, __uint_as_float(sv[c + 2]));
        t3 = fmaxf(t3, __uint_as_float(sv[c + 3]));
      }
      const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * scale;  // the scale is positive
      // the running maximum moves only when the true one is more than 2^8 ahead: P stays below 2^8,
      // and O needs rescaling on few tiles
      const float m_new = (tmax > m_run + RESCALE_STEP || m_run == -INFINITY) ? fmaxf(tmax, m_run) : m_run;
      const float alpha = m_new == m_run ? 1.f : ex2(m_run - m_new);  // 0 on a row's first visible tile
      m_run = m_new;
      const float neg_m = m_new == -INFINITY ? 0.f : -m_new;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        const float e0 = ex2(fmaf(__uint_as_float(sv[c]), scale, neg_m));
        const float e1 = ex2(fmaf(__uint_as_float(sv[c + 1]), scale, neg_m));
        const float e2 = ex2(fmaf(__uint_as_float(sv[c + 2]), scale, neg_m));
        const float e3 = ex2(fmaf(__uint_as_float(sv[c + 3]), scale, neg_m));
        a0 += e0;
        a1 += e1;
        a2 += e2;
        a3 += e3;
        pk[c / 2] = pack2(e0, e1);
        pk[c / 2 + 1] = pack2(e2, e3);
      }
      l_run = l_run * alpha + ((a0 + a1) + (a2 + a3));
      // the group's previous O[g] += P V must be complete before O[g] is rescaled and P[g] rewritten
      if (j > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(&o_done[g], (j - 1) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(o_addr + (uint32_t)c0, ov);
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
            tmem_st32(o_addr + (uint32_t)c0, ov);
          }
          tmem_st_wait();
        }
      }
      // P row r: 64 bfloat16 in the 32 columns of the group's A operand
      tmem_st32(p_addr, pk);
      // value rows no row of this tile may see: zero them (whole 128-byte rows, every slice)
      if (key0 < lo || key0 + BN - 1 > pos_last || bad != 0u) {
        if (!__all_sync(0xffffffffu, mbar_wait(&v_full[i % V_STAGES], (i / V_STAGES) & 1))) {
          ok = false;
          break;
        }
        const int key_row = r >> 1;  // two threads per key row
        const int key = key0 + key_row;
        bool dead = key > pos_last || key < lo;
        if (!dead) {
          const int pg = table[key / p.page_size];
          dead = pg < 0 || pg >= p.num_pages;
        }
        if (dead) {
          const uint32_t row_addr = smem_u32(v_s + (i % V_STAGES) * KV_BYTES) + (uint32_t)key_row * 128u +
                                    (uint32_t)(r & 1) * 64u;
#pragma unroll
          for (int h = 0; h < KD; ++h)
#pragma unroll
            for (int c = 0; c < 4; ++c) st_shared16(row_addr + h * KV_SLICE + c * 16, make_uint4(0, 0, 0, 0));
        }
        fence_async_smem();
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[g]);
    }
    // the group's last product
    if (ok && j > 0 && !__all_sync(0xffffffffu, mbar_wait(&o_done[g], (j - 1) & 1))) ok = false;
    if (!ok) failed = 1;
    if (g == 1) {
      merge_m[r] = m_run;
      merge_l[r] = l_run;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight softmax warps
    if (g == 0 && !failed) {
      // ---- merge the two groups' partial results (two key splits) and store row r
      tc_fence_after();
      const bool two = n_kt > 1;  // group 1 had tiles: O[1] holds its part
      const float m1 = two ? merge_m[r] : -INFINITY, l1 = two ? merge_l[r] : 0.f;
      const float M = fmaxf(m_run, m1);
      const float w0 = m_run == -INFINITY ? 0.f : ex2(m_run - M);
      const float w1 = m1 == -INFINITY ? 0.f : ex2(m1 - M);
      const float denom = l_run * w0 + l1 * w1;
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      const float f0 = w0 * inv, f1 = w1 * inv;
      bf16* dst = p.out;
      if (row_ok) dst = p.out + (size_t)(qs + tok0 + r / G) * p.out_stride + (size_t)(kvh * G + r % G) * D;
      // every lane takes part in the warp-wide loads of tensor memory; lanes without a row store nothing
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(lane_addr + (uint32_t)(O_COL + c0), ov);
        if (two) {
          uint32_t ow[32];
          tmem_ld32(lane_addr + (uint32_t)(O_COL + D + c0), ow);
#pragma unroll
          for (int c = 0; c < 32; ++c)
            ov[c] = __float_as_uint(__uint_as_float(ov[c]) * f0 + __uint_as_float(ow[c]) * f1);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * f0);
        }
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(ov[c]), __uint_as_float(ov[c + 1]));
            w.y = pack2(__uint_as_float(ov[c + 2]), __uint_as_float(ov[c + 3]));
            w.z = pack2(__uint_as_float(ov[c + 4]), __uint_as_float(ov[c + 5]));
            w.w = pack2(__uint_as_float(ov[c + 6]), __uint_as_float(ov[c + 7]));
            *reinterpret_cast<uint4*>(dst + c0 + c) = w;
          }
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0) atomicOr(p.err, DSP_ERR_WAIT_LIMIT);
    // let copies that are still on their way land before the shared memory goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// DISPEC_B200_PAGE_RUNS=0 in the environment keeps every page on a request of its own (for
// measurements, and for tests that compare the two ways of loading); read at every call.
bool page_runs_enabled() {
  const char* v = getenv("DISPEC_B200_PAGE_RUNS");
  return !(v != nullptr && v[0] == '0');
}

struct MapKey {
  const void* base;
  long num_pages;
  int heads, page_size;
  bool has_runs;
  CUtensorMap map, runs;
};
// tensor maps of the pools seen so far (a handful: two per layer cache): one whose box is a page of
// one head, and one whose box is a key tile's worth of consecutive pages (absent for a pool of
// fewer pages than a tile has)
bool pool_map(const void* base, long num_pages, int heads, int page_size, CUtensorMap* out, CUtensorMap* runs,
              bool* has_runs) {
  constexpr int SLOTS = 256;
  static MapKey cache[SLOTS];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].num_pages == num_pages && cache[i].heads == heads &&
        cache[i].page_size == page_size) {
      *out = cache[i].map;
      *runs = cache[i].runs;
      *has_runs = cache[i].has_runs;
      return true;
    }
  MapKey k;
  k.base = base;
  k.num_pages = num_pages;
  k.heads = heads;
  k.page_size = page_size;
  if (!make_map(&k.map, base, num_pages * heads * page_size, D, D, page_size)) return false;
  k.has_runs = make_map_page_runs(&k.runs, base, num_pages, heads, page_size, D, BN / page_size);
  if (!k.has_runs) k.runs = k.map;
  if (used < SLOTS) cache[used++] = k;
  *out = k.map;
  *runs = k.runs;
  *has_runs = k.has_runs;
  return true;
}
}  // namespace

// Attention of the tiles tile_offset .. tile_offset + num_tiles - 1 of the step's tile list (tiles of
// tokens_per_tile tokens, 128 / group size at most).  Returns 0, or: 1 launch failed, 2 unsupported
// head/group counts or page size (a power of two from 8 to 64), 3 misaligned operands, 4 the
// shared-memory opt-in or the tensor maps failed.
extern "C" int DSP_CAT(dsp_attn_tcgen05_d, DSP_HEAD_DIM)(
    const void* q, long q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int pt_stride, const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_tok0,
    int tile_offset, int num_tiles, void* out, long out_stride, int H, int KVH, int tokens_per_tile,
    int page_size, int num_pages, int window, float scale, int* err, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (KVH <= 0 || H % KVH != 0 || (H / KVH) * tokens_per_tile > BM || tokens_per_tile < 1 || KVH > 65535) return 2;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 2;
  if (!(scale > 0.f)) return 2;
  if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)q % 16) || ((uintptr_t)k_pool % 16) ||
      ((uintptr_t)v_pool % 16) || ((uintptr_t)out % 16))
    return 3;
  Params p;
  p.q = (const bf16*)q;
  p.q_stride = q_stride;
  p.page_table = page_table;
  p.pt_stride = pt_stride;
  p.q_start = q_start;
  p.ctx_len = ctx_len;
  p.tile_seq = tile_seq;
  p.tile_tok0 = tile_tok0;
  p.out = (bf16*)out;
  p.out_stride = out_stride;
  p.H = H;
  p.KVH = KVH;
  p.G = H / KVH;
  p.tokens_per_tile = tokens_per_tile;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = err;
  CUtensorMap map_k, map_v, runs_k, runs_v;
  bool has_runs_k = false, has_runs_v = false;
  if (!pool_map(k_pool, num_pages, KVH, page_size, &map_k, &runs_k, &has_runs_k) ||
      !pool_map(v_pool, num_pages, KVH, page_size, &map_v, &runs_v, &has_runs_v))
    return 4;
  p.page_runs = has_runs_k && has_runs_v && page_runs_enabled();
  static bool configured = false;  // once; not repeated under graph capture
  if (!configured) {
    if (cudaFuncSetAttribute(attn_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return 4;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tiles, KVH, 1);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = (size_t)SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, attn_tcgen05_kernel, p, tile_offset, map_k, map_v, runs_k, runs_v) == cudaSuccess ? 0 : 1;
}
