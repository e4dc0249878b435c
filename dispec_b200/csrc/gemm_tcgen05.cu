// C[M,N] = A[M,K] * W[N,K]^T (+ bias) (+ residual) for many rows (prefill), bfloat16 in, 32-bit
// accumulation on the fifth-generation tensor cores.
//
// Persistent: one CTA per SM walks over 128 x 256 tiles of C.  A and W tiles of 64 k (128 bytes a
// row) come by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a four-stage ring
// in shared memory that never drains between tiles; one thread issues tcgen05.mma (M 128, N 256,
// K 16, operands described by shared-memory descriptors, K-major) into one of two 128-lane x
// 256-column accumulators in tensor memory; tcgen05.commit hands each stage back to the TMA
// thread through an mbarrier and, after a tile's last k block, tells the four epilogue warps that
// the accumulator is complete.  They read it with tcgen05.ld (each warp its own 32 lanes), add
// bias and residual in 32-bit, round once and store, while the products of the next tile already
// run into the other accumulator.
//
// Every wait on an mbarrier is bounded: if it runs out, the kernel records it in the device error
// word, lets copies in flight land, frees its tensor memory and returns.
#include "tcgen05_common.cuh"

namespace {
using namespace tc;
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;  // two accumulators of 256 columns
// warp 0: TMA, warp 1: MMA and tensor-memory allocation, warps 2-5: epilogue (a warp reaches the 32
// lanes of tensor memory that its index modulo 4 names).  Eight epilogue warps, two per quarter taking
// the chunks of columns in turn, left every product alone as fast as four (gate/up 92 us either way:
// the products, not the epilogue, bound it) and made the prefill step 18 % slower.
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 32 * (2 + EPI_WARPS);

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

struct Epilogue {
  int epilogue;
  const bf16* bias;
  const void* residual;
  long ldr;
  void* C;
  long ldc;
  int M, N, K;
  int k_boxes;  // the tensor maps are the three-dimensional ones: one request brings SUB k blocks (pair kernel)
};

// silu(gate) * up of the bfloat16 model on the hardware's exponential and reciprocal (a few units in
// the last place of 32 bits, far below the output's rounding): four epilogue warps, one per
// scheduler, run 128 of these per thread and tile, and their length in instructions is their time
__device__ __forceinline__ float silu_times(float gate, float up) {
  return __fdividef(gate, 1.f + __expf(-gate)) * up;
}

template <typename TOut>
__device__ __forceinline__ void store_row_chunk(const Epilogue& e, const uint32_t (&v)[32], int row, int col) {
  if (row >= e.M || col >= e.N) return;
  if (e.epilogue == EPI_SWIGLU) {
    // W rows alternate in blocks of 16: this chunk holds 16 gates and the 16 ups of the same outputs
    if (col + 32 > e.N) return;
    TOut* dst = reinterpret_cast<TOut*>(e.C) + (size_t)row * e.ldc + (col >> 1);
    if (sizeof(TOut) == 2 && ((uintptr_t)dst % 16) == 0) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint4 oraw;
        bf16* ob = reinterpret_cast<bf16*>(&oraw);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float g = __uint_as_float(v[j * 8 + t]), u = __uint_as_float(v[16 + j * 8 + t]);
          ob[t] = __float2bfloat16(silu_times(g, u));
        }
        reinterpret_cast<uint4*>(dst)[j] = oraw;
      }
    } else {
#pragma unroll  // constant indices: the accumulators stay in registers
      for (int t = 0; t < 16; ++t) {
        const float g = __uint_as_float(v[t]), u = __uint_as_float(v[16 + t]);
        dst[t] = from_f32<TOut>(silu_times(g, u));
      }
    }
    return;
  }
  TOut* dst = reinterpret_cast<TOut*>(e.C) + (size_t)row * e.ldc + col;
  const TOut* res = e.residual ? reinterpret_cast<const TOut*>(e.residual) + (size_t)row * e.ldr + col : nullptr;
  const int valid = min(32, e.N - col);
  if (valid == 32 && sizeof(TOut) == 2 && (((uintptr_t)dst | (uintptr_t)res) % 16) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 rraw = make_uint4(0u, 0u, 0u, 0u);
      if (res) rraw = reinterpret_cast<const uint4*>(res)[j];
      const bf16* rb = reinterpret_cast<const bf16*>(&rraw);
      uint4 oraw;
      bf16* ob = reinterpret_cast<bf16*>(&oraw);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        float x = __uint_as_float(v[j * 8 + t]);
        if (e.bias) x += __bfloat162float(e.bias[col + j * 8 + t]);
        if (res) x += __bfloat162float(rb[t]);
        ob[t] = __float2bfloat16(x);
      }
      reinterpret_cast<uint4*>(dst)[j] = oraw;
    }
  } else {
#pragma unroll  // constant indices: a loop up to `valid` would put the accumulators into local memory on every path
    for (int t = 0; t < 32; ++t) {
      if (t < valid) {
        float x = __uint_as_float(v[t]);
        if (e.bias) x += __bfloat162float(e.bias[col + t]);
        if (res) x += to_f32(res[t]);
        dst[t] = from_f32<TOut>(x);
      }
    }
  }
}

template <typename TOut>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const Epilogue e, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1024 bytes
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t accum_full[2];
  __shared__ __align__(8) uint64_t accum_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (e.K + BK - 1) / BK;
  const int n_tiles = (e.N + BN - 1) / BN, m_tiles = (e.M + BM - 1) / BM;
  const int num_tiles = n_tiles * m_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accum_full[b], 1);
      mbar_init(&accum_empty[b], EPI_WARPS);  // one arrival per epilogue warp
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: the ring runs on across tiles
    if (lane == 0) {
      // The weights do not depend on the kernel before: the first ring of W tiles is asked for
      // while that kernel still runs.  A comes from it, so A waits.
      const int ahead = num_kb < STAGES ? num_kb : STAGES;
      for (int kb = 0; kb < ahead; ++kb) {
        mbar_expect_tx(&full_bar[kb], STAGE_BYTES);
        tma_load_2d(smem + kb * STAGE_BYTES + A_BYTES, &map_w, &full_bar[kb], kb * BK,
                    ((int)blockIdx.x % n_tiles) * BN);
      }
      pdl_wait();
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
        const int m0 = (tile / n_tiles) * BM, n0 = (tile % n_tiles) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          unsigned char* a_dst = smem + s * STAGE_BYTES;
          if (it >= ahead) {
            if (!mbar_wait(&empty_bar[s], phase ^ 1)) {
              failed = 1;
              break;
            }
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(a_dst + A_BYTES, &map_w, &full_bar[s], kb * BK, n0);
          }
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * BK, m0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, BN);
      int it = 0, local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have emptied this accumulator (two tiles ago)
        if (!mbar_wait(&accum_empty[buf], ((local >> 1) & 1) ^ 1)) {
          failed = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], phase)) {
            failed = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // the next 16 k of a 128-byte swizzled row: 32 bytes further
            umma(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[s]);  // the stage is free once these products have read it
        }
        if (failed) break;
        umma_commit(&accum_full[buf]);
      }
    }
  } else {
    // ---- epilogue warps 2..5: warp w owns accumulator lanes 32 (w % 4) .. +31
    pdl_wait();  // the residual comes from earlier kernels, and C may still be read by them
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile / n_tiles) * BM, n0 = (tile % n_tiles) * BN;
      // every lane waits (the barrier's completion orders its own reads); the warp decides as one
      if (!__all_sync(0xffffffffu, mbar_wait(&accum_full[buf], (local >> 1) & 1))) {
        failed = 1;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      for (int c0 = 32 * ((warp - 2) >> 2); c0 < BN; c0 += 32 * (EPI_WARPS / 4)) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), v);
        store_row_chunk<TOut>(e, v, row, n0 + c0);
      }
      // the accumulator has been read: hand it back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&accum_empty[buf])) : "memory");
    }
  }

  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_WAIT_LIMIT);
    // let copies that are still on their way land before the shared memory goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------
// The same product on CTA pairs (cta_group::2): a cluster of two CTAs computes a 256 x 256 tile.
// Each CTA loads its own 128 rows of A and its own 128 rows (half) of the W tile, so a k block
// costs 32 KB of shared-memory traffic per CTA instead of 48 KB and the ring is six stages deep;
// the leader CTA's thread issues tcgen05.mma.cta_group::2 (M 256) for both, which reads the two
// halves of the W tile from both CTAs' shared memory and writes each CTA's 128 rows into its own
// tensor memory.  Both CTAs' TMA loads complete on the leader's "full" barrier; tcgen05.commit
// with multicast frees the stage in both CTAs and announces the finished accumulator to both;
// both CTAs' epilogue warps arrive on the leader's "accumulator empty" barrier.  No TMA load is
// multicast.
// What a chunk of 32 outputs of a row needs beside its accumulators, asked for before they arrive:
// in the loop "accumulators of the chunk, then its bias and residual, then the stores", every
// chunk paid the latency of tensor memory and then that of global memory (1,200 to 1,500 cycles a
// chunk; 5 us for the one tile of a CTA pair in the three narrow products of a layer).
struct ChunkOperands {
  uint4 res[4];
  uint4 bias[4];
  bool fast;  // bfloat16 output, a whole chunk inside the matrix, 16-byte aligned operands
};
template <typename TOut>
__device__ __forceinline__ void fetch_chunk_operands(const Epilogue& e, int row, int col, ChunkOperands& op) {
  op.fast = false;
  if (sizeof(TOut) != 2 || e.epilogue != EPI_PLAIN || row >= e.M || col + 32 > e.N) return;
  const TOut* dst = reinterpret_cast<const TOut*>(e.C) + (size_t)row * e.ldc + col;
  const TOut* res = e.residual ? reinterpret_cast<const TOut*>(e.residual) + (size_t)row * e.ldr + col : nullptr;
  const bf16* bias = e.bias ? e.bias + col : nullptr;
  if ((((uintptr_t)dst | (uintptr_t)res | (uintptr_t)bias) % 16) != 0) return;
  op.fast = true;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    op.res[j] = res ? reinterpret_cast<const uint4*>(res)[j] : make_uint4(0u, 0u, 0u, 0u);
    op.bias[j] = bias ? __ldg(reinterpret_cast<const uint4*>(bias) + j) : make_uint4(0u, 0u, 0u, 0u);
  }
}
// The chunk's outputs from its accumulators and the operands fetched before; the sums are formed
// as in store_row_chunk: accumulator + bias + residual in 32 bits, rounded once.
template <typename TOut>
__device__ __forceinline__ void store_row_chunk_with(const Epilogue& e, const uint32_t (&v)[32], int row, int col,
                                                     const ChunkOperands& op) {
  if (!op.fast) {
    store_row_chunk<TOut>(e, v, row, col);
    return;
  }
  bf16* dst = reinterpret_cast<bf16*>(e.C) + (size_t)row * e.ldc + col;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bf16* rb = reinterpret_cast<const bf16*>(&op.res[j]);
    const bf16* bb = reinterpret_cast<const bf16*>(&op.bias[j]);
    uint4 oraw;
    bf16* ob = reinterpret_cast<bf16*>(&oraw);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      float x = __uint_as_float(v[j * 8 + t]);
      if (e.bias) x += __bfloat162float(bb[t]);
      if (e.residual) x += __bfloat162float(rb[t]);
      ob[t] = __float2bfloat16(x);
    }
    reinterpret_cast<uint4*>(dst)[j] = oraw;
  }
}

constexpr int STAGES2 = 3;   // ring slots of the pair kernel, SUB k blocks each
constexpr int SUB = 2;       // k blocks per ring slot: one barrier round trip of the issuing thread per 128 of k
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;       // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(leader_bar) & PEER_BIT_MASK), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint64_t* leader_bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(leader_bar) & PEER_BIT_MASK), "r"(c0), "r"(c1),
        "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
        "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_on_leader(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(smem_u32(bar)), "r"(0u)
      : "memory");
}

template <typename TOut, int BNP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const Epilogue e, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES2];   // used in the leader: both CTAs' loads land here
  __shared__ __align__(8) uint64_t empty_bar[STAGES2];  // one per CTA, freed by the multicast commit
  __shared__ __align__(8) uint64_t accum_full[2];       // one per CTA
  __shared__ __align__(8) uint64_t accum_empty[2];      // used in the leader: both CTAs' epilogue warps arrive
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int num_kb = (e.K + BK - 1) / BK;
  constexpr int B_HALF = (BNP / 2) * BK * 2;   // this CTA's half of the W tile, one k block
  constexpr int STAGE_P = A_BYTES + B_HALF;    // one k block of both operands
  const int n_tiles = (e.N + BNP - 1) / BNP, m_tiles = (e.M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = n_tiles * m_tiles;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accum_full[b], 1);
      mbar_init(&accum_empty[b], 2 * EPI_WARPS);
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // as in the one-CTA kernel: the first ring of W tiles is asked for before the wait.  A ring
      // slot holds SUB k blocks of A, then SUB k blocks of this CTA's half of W; with the
      // three-dimensional maps one request brings all SUB blocks of an operand (and counts the
      // bytes of all SUB, zero-filled beyond K), else one request per k block
      const int num_steps = (num_kb + SUB - 1) / SUB;  // ring slots per tile
      const int ahead = num_steps < STAGES2 ? num_steps : STAGES2;
      auto slot_bytes = [&](int st) {
        const int subs = num_kb - st * SUB < SUB ? num_kb - st * SUB : SUB;
        return 2 * STAGE_P * (e.k_boxes ? SUB : subs);
      };
      auto load_w = [&](unsigned char* slot, uint64_t* bar, int st, int w0) {
        unsigned char* dst = slot + SUB * A_BYTES;
        if (e.k_boxes) {
          tma_load_3d_pair(dst, &map_w, bar, 0, w0, st * SUB);
        } else {
          for (int u = 0; u < SUB && st * SUB + u < num_kb; ++u)
            tma_load_2d_pair(dst + u * B_HALF, &map_w, bar, (st * SUB + u) * BK, w0);
        }
      };
      auto load_a = [&](unsigned char* slot, uint64_t* bar, int st, int m0) {
        if (e.k_boxes) {
          tma_load_3d_pair(slot, &map_a, bar, 0, m0, st * SUB);
        } else {
          for (int u = 0; u < SUB && st * SUB + u < num_kb; ++u)
            tma_load_2d_pair(slot + u * A_BYTES, &map_a, bar, (st * SUB + u) * BK, m0);
        }
      };
      for (int st = 0; st < ahead; ++st) {
        if (rank == 0) mbar_expect_tx(&full_bar[st], slot_bytes(st));
        load_w(smem + st * SUB * STAGE_P, &full_bar[st], st, ((pair / m_tiles) % n_tiles) * BNP + (int)rank * (BNP / 2));
      }
      pdl_wait();
      int it = 0;
      for (int tile = pair; tile < num_tiles && !failed; tile += num_pairs) {
        const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM;
        const int w0 = (tile / m_tiles) * BNP + (int)rank * (BNP / 2);
        for (int st = 0; st < num_steps; ++st, ++it) {
          const int s = it % STAGES2;
          const uint32_t phase = (it / STAGES2) & 1;
          unsigned char* slot = smem + s * SUB * STAGE_P;
          if (it >= ahead) {
            if (!mbar_wait(&empty_bar[s], phase ^ 1)) {
              failed = 1;
              break;
            }
            if (rank == 0) mbar_expect_tx(&full_bar[s], slot_bytes(st));
            load_w(slot, &full_bar[s], st, w0);
          }
          load_a(slot, &full_bar[s], st, m0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2 * BM, BNP);  // M 256 across the pair
      int it = 0, local = 0;
      for (int tile = pair; tile < num_tiles && !failed; tile += num_pairs, ++local) {
        const int buf = local & 1;
        if (!mbar_wait(&accum_empty[buf], ((local >> 1) & 1) ^ 1)) {
          failed = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * 256);
        const int num_steps = (num_kb + SUB - 1) / SUB;
        for (int st = 0; st < num_steps; ++st, ++it) {
          const int s = it % STAGES2;
          const uint32_t phase = (it / STAGES2) & 1;
          if (!mbar_wait(&full_bar[s], phase)) {
            failed = 1;
            break;
          }
          tc_fence_after();
          const int subs = num_kb - st * SUB < SUB ? num_kb - st * SUB : SUB;
          for (int u = 0; u < subs; ++u) {
            const uint32_t a_addr = smem_u32(smem + s * SUB * STAGE_P + u * A_BYTES);
            const uint32_t b_addr = smem_u32(smem + s * SUB * STAGE_P + SUB * A_BYTES + u * B_HALF);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_pair(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (st | u | k) != 0);
          }
          umma_commit_pair(&empty_bar[s]);
        }
        if (failed) break;
        umma_commit_pair(&accum_full[buf]);
      }
    }
  } else {
    pdl_wait();  // the residual comes from earlier kernels, and C may still be read by them
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM, n0 = (tile / m_tiles) * BNP;
      if (!__all_sync(0xffffffffu, mbar_wait(&accum_full[buf], (local >> 1) & 1))) {
        failed = 1;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      // two chunks in flight: while one is turned into outputs, the accumulators, the bias and
      // the residual of the next are on their way
      static_assert(BNP % 64 == 0 && EPI_WARPS == 4, "chunks are taken in pairs by four warps");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 256);
      uint32_t va[32], vb[32];
      ChunkOperands oa, ob;
      tmem_ld32_nowait(taddr, va);
      fetch_chunk_operands<TOut>(e, row, n0, oa);
#pragma unroll 1
      for (int c0 = 0; c0 < BNP; c0 += 64) {
        tmem_ld_wait();
        tmem_ld32_nowait(taddr + (uint32_t)(c0 + 32), vb);
        fetch_chunk_operands<TOut>(e, row, n0 + c0 + 32, ob);
        store_row_chunk_with<TOut>(e, va, row, n0 + c0, oa);
        tmem_ld_wait();
        if (c0 + 64 < BNP) {
          tmem_ld32_nowait(taddr + (uint32_t)(c0 + 64), va);
          fetch_chunk_operands<TOut>(e, row, n0 + c0 + 64, oa);
        }
        store_row_chunk_with<TOut>(e, vb, row, n0 + c0 + 32, ob);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_on_leader(&accum_empty[buf]);
    }
  }

  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_WAIT_LIMIT);
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  cluster_sync_all();  // the peer is done with this CTA's shared memory and barriers
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

// bfloat16 A [M, K] (row stride lda) and W [N, K] (contiguous); C and residual bfloat16 or float32.
// epilogue 1: SwiGLU over W rows alternating in blocks of 16 (16 gate rows, their 16 up rows):
// C is [M, N/2], no bias, no residual.
extern "C" int dsp_gemm_tcgen05(const void* A, long lda, const void* W, const void* bias, const void* residual,
                                long ldr, void* C, long ldc, int M, int N, int K, int out_dtype, int pair_mode,
                                int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DSP_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0, "dsp_gemm_tcgen05: K=%d and the row stride must be multiples of 8", K);
  DSP_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0, "dsp_gemm_tcgen05: operands must be 16-byte aligned");
  DSP_REQUIRE(out_dtype == DSP_BF16 || out_dtype == DSP_F32, "dsp_gemm_tcgen05: unknown output dtype %d", out_dtype);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_gemm_tcgen05: no device error word");
  CUtensorMap map_a, map_w;  // encoded below, once the tile shape is known (an encoding costs the host a microsecond)
  DSP_REQUIRE(epilogue == EPI_PLAIN || (N % 32 == 0 && bias == nullptr && residual == nullptr),
              "dsp_gemm_tcgen05: the SwiGLU epilogue needs N in whole blocks of 32 and no bias or residual");
  Epilogue e;
  e.epilogue = epilogue;
  e.bias = (const bf16*)bias;
  e.residual = residual;
  e.ldr = ldr;
  e.C = C;
  e.ldc = ldc;
  e.M = M;
  e.N = N;
  e.K = K;
  e.k_boxes = 0;
  const int smem = STAGES * STAGE_BYTES + 1024;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    DSP_CUDA(cudaGetDevice(&dev));
    DSP_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  if (pair_mode) {
    // tile width: 256, or 192 when that puts more of the CTA pairs to work in the last round
    // (cost ~ rounds x width; N 1536 on 74 pairs: 48 tiles of 256 against 64 tiles of 192)
    const long pairs_avail = num_sms / 2;
    const long m_tiles2 = (M + 2 * BM - 1) / (2 * BM);
    auto cost = [&](int bn) {
      const long tiles2 = (long)((N + bn - 1) / bn) * m_tiles2;
      return ((tiles2 + pairs_avail - 1) / pairs_avail) * bn;
    };
    const int bnp = cost(192) < cost(256) ? 192 : 256;
    e.k_boxes = (make_map_k_blocks(&map_a, A, M, K, lda, BM, SUB) && make_map_k_blocks(&map_w, W, N, K, K, bnp / 2, SUB)) ? 1 : 0;
    if (!e.k_boxes) {
      DSP_REQUIRE(make_map(&map_a, A, M, K, lda, BM), "dsp_gemm_tcgen05: cannot encode the tensor map of A");
      DSP_REQUIRE(make_map(&map_w, W, N, K, K, bnp / 2), "dsp_gemm_tcgen05: cannot encode the tensor map of W");
    }
    const int smem2 = STAGES2 * SUB * (A_BYTES + (bnp / 2) * BK * 2) + 1024;
    const long tiles2 = (long)((N + bnp - 1) / bnp) * m_tiles2;
    const long pairs = tiles2 < pairs_avail ? tiles2 : pairs_avail;
    dim3 grid2((unsigned)(2 * pairs));
#define DSP_LAUNCH_PAIR(TYPE, WIDTH)                                                                          \
  do {                                                                                                       \
    static bool configured = false;                                                                          \
    if (!configured) {                                                                                       \
      DSP_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<TYPE, WIDTH>,                                   \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));                    \
      prefer_max_shared(reinterpret_cast<const void*>(gemm_tcgen05_pair_kernel<TYPE, WIDTH>));               \
      configured = true;                                                                                     \
    }                                                                                                        \
    launch_pdl(gemm_tcgen05_pair_kernel<TYPE, WIDTH>, grid2, dim3(THREADS), smem2, stream, map_a, map_w,     \
               e, err);                                                                                      \
  } while (0)
    if (out_dtype == DSP_BF16) {
      if (bnp == 192) DSP_LAUNCH_PAIR(bf16, 192); else DSP_LAUNCH_PAIR(bf16, 256);
    } else {
      if (bnp == 192) DSP_LAUNCH_PAIR(float, 192); else DSP_LAUNCH_PAIR(float, 256);
    }
#undef DSP_LAUNCH_PAIR
    DSP_CHECK_LAUNCH("dsp_gemm_tcgen05 (CTA pairs)");
    return 0;
  }
  DSP_REQUIRE(make_map(&map_a, A, M, K, lda, BM), "dsp_gemm_tcgen05: cannot encode the tensor map of A");
  DSP_REQUIRE(make_map(&map_w, W, N, K, K, BN), "dsp_gemm_tcgen05: cannot encode the tensor map of W");
  const long tiles = (long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  dim3 grid((unsigned)(tiles < num_sms ? tiles : num_sms));
  if (out_dtype == DSP_BF16) {
    static bool configured = false;
    if (!configured) {
      DSP_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured = true;
    }
    launch_pdl(gemm_tcgen05_kernel<bf16>, dim3(grid), dim3(THREADS), smem, stream, map_a, map_w, e, err);
  } else {
    static bool configured = false;
    if (!configured) {
      DSP_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured = true;
    }
    launch_pdl(gemm_tcgen05_kernel<float>, dim3(grid), dim3(THREADS), smem, stream, map_a, map_w, e, err);
  }
  DSP_CHECK_LAUNCH("dsp_gemm_tcgen05");
  return 0;
}
