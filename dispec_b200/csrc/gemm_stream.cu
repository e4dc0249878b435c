// C[M,N] = A[M,K] * W[N,K]^T (+ bias) (+ residual) for up to 128 rows of A, bfloat16 in, 32-bit
// accumulation: the matrix product of decoding, bound by streaming W once from HBM, on TMA and
// the fifth-generation tensor cores.
//
// Roles are swapped: 128 rows of W are the M side of tcgen05.mma, the few rows of A (padded to
// 16, 32, 64 or 128) its N side, so the accumulator in tensor memory is 128 lanes (rows of W) by a
// few columns (rows of A).  One thread streams W tiles of 128 rows x 64 k (16 KB a request)
// and the matching slice of A by TMA into a ring of 4 to 5 stages (two CTAs per SM, about 180 KB
// on its way per SM, which plain loads cannot keep in flight); one thread issues the products; four warps read
// the accumulator, apply the epilogue and store.  With programmatic dependent launch the first
// W tiles are requested before the kernel waits for its predecessor.
//
// K is split across a thread-block cluster (up to 8 CTAs) when there are too few 128-row blocks
// of W to fill the SMs, and the partial tiles are added through distributed shared memory in rank
// order (deterministic, no global scratch): every CTA sends each row of its partial tile to the
// CTA that finishes that row (remote stores that count their bytes on a barrier of the receiver)
// and adds what arrived in its own memory; no remote read, and no CTA waits for the others
// before it leaves: whole rows travel 16 bytes a lane.  Up to 16 rows of A the inbox lies behind
// the ring and nobody waits for the cluster at all; with more rows the inbox is part of the
// drained ring, which costs one cluster barrier.  Without a split a CTA walks over several
// blocks of W and the accumulator is double-buffered, so the epilogue of one block overlaps the
// next.
//
// Epilogues: bias[n], residual[m, n] (32-bit sum, rounded once), or SwiGLU over W rows that
// alternate in blocks of 16 (16 gate rows, the 16 up rows of the same outputs): C is [M, N/2].
// Every wait on an mbarrier is bounded; a wait that runs out is recorded in the device error word.
#include <cooperative_groups.h>

#include "tcgen05_common.cuh"

namespace cg = cooperative_groups;

namespace {
using namespace tc;
constexpr int ROWS_W = 128, BK = 64, UMMA_K = 16;
constexpr int W_BYTES = ROWS_W * BK * 2;
// warp 0: TMA; then ISSUERS warps whose first lanes issue the products (the first of them also owns
// the tensor memory); then four epilogue warps
constexpr int MAX_SPLITS = 8;
enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

template <int NB> struct Cfg {
  static constexpr int X_BYTES = NB * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  // about 100 KB of ring per CTA, so that two CTAs fit an SM: the next kernel's CTA (programmatic
  // dependent launch) fills its ring with W while this kernel's CTA is still streaming
  static constexpr int STAGES = NB == 16 ? 5 : NB == 32 ? 5 : NB == 64 ? 4 : 5;  // 128 rows of A: one CTA per SM
  // One thread's turn of the ring (wait for the stage, fence, four products, commit) takes about
  // 0.3 us, of which the tensor pipe is busy a third (a product of 128 x 16 x 16 every 55 cycles from
  // one issuing thread, every 39 from two: `bench.py --only mma-rate`); a W tile of 16 KB per 0.3 us is
  // 55 GB/s, which is what an SM's share of the memory bandwidth delivers.  The four k steps of a k
  // block therefore belong to ISSUERS threads of different warps, each with a partial accumulator of
  // its own, so that their turns overlap; the epilogue adds the partial accumulators up in a fixed
  // order.  Measured on the captured decode step at 8 rows: first stage to last product 0.96 -> 0.7 us
  // on the small products, 8.1 -> 7.6 us on gate/up, 5.75 -> 4.7 us on down.  (Whole k blocks dealt
  // to five issuers that own a stage of the ring each measured 1 % slower on the whole step.)  Two
  // CTAs share the SM's 512 columns of tensor memory.
  // (at 128 rows of A a product of 128 x 128 x 16 keeps the pipe busy for the 64 cycles one thread
  // needs to issue it: one issuer, no partial accumulators)
  static constexpr int PARTS = NB == 16 ? 4 : NB <= 64 ? 2 : 1;
  static constexpr int ISSUERS = PARTS;
  static constexpr int FIRST_EPI_WARP = 1 + ISSUERS;
  static constexpr int THREADS = 32 * (1 + ISSUERS + 4);
  static constexpr int MIN_CTAS = NB <= 64 ? 2 : 1;  // CTAs per SM the registers are held down for
  // the epilogue takes the accumulator in windows of at most 64 columns (rows of A): what a thread holds at once
  static constexpr int WINDOW = NB <= 64 ? NB : 64;
  static constexpr int ACC_COLS = PARTS * NB;  // one accumulator buffer
  static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  // K split over a cluster: every CTA sends the rows of its partial tile to the CTA that finishes
  // them (row m to rank m % splits), into an inbox of [source rank][rows per CTA][128] floats.  Up
  // to 16 rows of A (at most 16 + 8 rows of inbox) it has room of its own behind the ring
  static constexpr bool PUSH = NB == 16;
  // behind the ring: that inbox, or 8 KB in which, without a split of K, an epilogue warp turns 16
  // columns of its accumulator around, so that a lane stores four outputs of one row
  static constexpr int INBOX_BYTES = PUSH ? (16 + MAX_SPLITS) * ROWS_W * 4 : 4 * 16 * 32 * 4;
};

// Timestamps for measurements, compiled in only with -DDSP_STAMPS (DISPEC_B200_STAMPS=1 at build
// time): every CTA of a launch records the global timer at up to twelve points of its life.
#ifdef DSP_STAMPS
__device__ unsigned long long g_stamps[1 << 21];
#define STAMP(pt)                                                                                      \
  do {                                                                                                 \
    if (a.stamp_base >= 0) {                                                                           \
      unsigned long long t__;                                                                          \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                          \
      g_stamps[(size_t)a.stamp_base + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 12 + (pt)] = t__; \
    }                                                                                                  \
  } while (0)
#else
#define STAMP(pt)
#endif

struct Args {
  long stamp_base;  // first slot of this launch's timestamps, or -1
  const bf16* bias;
  const void* residual;
  long ldr;
  void* C;
  long ldc;
  int M, N, K;
  int kb_per_split;
  int epilogue;
  // when the next kernel may start (programmatic dependent launch): 0 at once, 1 when this CTA has
  // requested its last tile of W
  int late_trigger;
  int vec4;  // rows and pointers allow stores of four outputs (N, row strides: multiples of 4; 16-byte pointers)
  // A norm around the product, split over two kernels (both null: none).  norm_src: the rows whose
  // mean square scales this product's rows, C = (A W^T) * rsqrt(mean(norm_src[m]^2) + norm_eps) + ...,
  // A being those rows times the norm's gain.  gain2, C2: a second output, the rounded result times
  // gain2[n], which is such an A for the product after this one.
  const bf16* norm_src;
  long ld_src;
  float norm_eps;
  const bf16* gain2;
  void* C2;
  long ldc2;
};

template <typename TOut>
__device__ __forceinline__ void finish(const Args& a, float v, int m, int n) {
  if (a.bias) v += __bfloat162float(a.bias[n]);
  if (a.residual) v += to_f32(reinterpret_cast<const TOut*>(a.residual)[(size_t)m * a.ldr + n]);
  const TOut out = from_f32<TOut>(v);
  reinterpret_cast<TOut*>(a.C)[(size_t)m * a.ldc + n] = out;
  if (a.C2)
    reinterpret_cast<TOut*>(a.C2)[(size_t)m * a.ldc2 + n] = from_f32<TOut>(to_f32(out) * __bfloat162float(a.gain2[n]));
}

// silu(gate) * up for the bfloat16 model.  One warp per scheduler runs the epilogue, so its length
// in instructions is its time: the hardware's exponential and reciprocal (a few units in the last
// place of 32 bits, far below the output's rounding) instead of the library's sequences, which at
// 64 rows of A made the epilogue of the gate/up product 3.9 us long.
__device__ __forceinline__ float silu_times(float gate, float up) {
  return __fdividef(gate, 1.f + __expf(-gate)) * up;
}

// four consecutive values of a row, as 32-bit floats
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
// what a store of the output type leaves of four 32-bit values
template <typename T> __device__ __forceinline__ float4 rounded4(float4 v) {
  return make_float4(to_f32(from_f32<T>(v.x)), to_f32(from_f32<T>(v.y)), to_f32(from_f32<T>(v.z)),
                     to_f32(from_f32<T>(v.w)));
}

// sum of the squares of eight bfloat16 values
__device__ __forceinline__ float square_sum8(const uint4 u) {
  const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float lo = __uint_as_float(w4[e] << 16), hi = __uint_as_float(w4[e] & 0xffff0000u);
    ss += lo * lo;
    ss += hi * hi;
  }
  return ss;
}

// The accumulator of this thread's W row: the partial accumulators added in a fixed order.
// NB columns from taddr on; the PARTS partial accumulators lie part_stride columns apart.
template <int NB, int PARTS>
__device__ __forceinline__ void load_accumulator(uint32_t taddr, uint32_t part_stride, uint32_t (&v)[NB]) {
  if constexpr (NB == 16) {
    // the partial accumulators lie side by side: one load of PARTS x 16 columns, one wait
    static_assert(PARTS == 4 || PARTS == 2, "loads of 32 or 64 columns");
    uint32_t all[PARTS * 16];
    if constexpr (PARTS == 4) {
      tmem_ld32_nowait(taddr, reinterpret_cast<uint32_t(&)[32]>(all[0]));
      tmem_ld32_nowait(taddr + 32, reinterpret_cast<uint32_t(&)[32]>(all[32]));
      tmem_ld_wait();
    } else {
      tmem_ld32(taddr, reinterpret_cast<uint32_t(&)[32]>(all[0]));
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float sum = __uint_as_float(all[c]);
#pragma unroll
      for (int p = 1; p < PARTS; ++p) sum += __uint_as_float(all[p * 16 + c]);
      v[c] = __float_as_uint(sum);
    }
  } else if constexpr (PARTS == 1) {
#pragma unroll
    for (int c0 = 0; c0 < NB; c0 += 32) tmem_ld32_nowait(taddr + (uint32_t)c0, reinterpret_cast<uint32_t(&)[32]>(v[c0]));
    tmem_ld_wait();
  } else {
    // 32 columns of every partial accumulator per trip to the tensor memory (a load and its wait
    // take a few hundred nanoseconds: they are not taken one after the other)
    static_assert(PARTS == 2, "two partial accumulators");
#pragma unroll
    for (int c0 = 0; c0 < NB; c0 += 32) {
      uint32_t part[32];
      tmem_ld32_nowait(taddr + (uint32_t)c0, reinterpret_cast<uint32_t(&)[32]>(v[c0]));
      tmem_ld32_nowait(taddr + part_stride + (uint32_t)c0, part);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c0 + c] = __float_as_uint(__uint_as_float(v[c0 + c]) + __uint_as_float(part[c]));
    }
  }
}

template <int NB, typename TOut>
__global__ void __launch_bounds__(Cfg<NB>::THREADS, Cfg<NB>::MIN_CTAS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const Args a, int* err) {
  using C = Cfg<NB>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[C::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
  __shared__ __align__(8) uint64_t accum_full[2];
  __shared__ __align__(8) uint64_t accum_empty[2];
  __shared__ __align__(8) uint64_t inbox_bar;  // counts the bytes of partial rows other ranks send here
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  if (threadIdx.x == 0) STAMP(0);  // entry
  if (!a.late_trigger) pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = gridDim.y, split = blockIdx.y;
  const int n_blocks = (a.N + ROWS_W - 1) / ROWS_W;
  const int kb_total = (a.K + BK - 1) / BK;
  const int kb_begin = split * a.kb_per_split;
  const int kb_end = min(kb_total, kb_begin + a.kb_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], C::ISSUERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accum_full[b], C::ISSUERS);
      mbar_init(&accum_empty[b], 4);
    }
    mbar_init(&inbox_bar, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the first issuer warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // first half of a cluster barrier: by the time a CTA sends its partial rows, every CTA of its
  // cluster has started (its shared memory is there)
  if (C::PUSH && splits > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // the CTA's work as one flat sequence of (block of W, k block) items
      const int my_tiles = blockIdx.x < n_blocks ? (n_blocks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const int total = my_tiles * num_kb;
      const int first = total < C::STAGES ? total : C::STAGES;
      auto w_row = [&](int it) { return ((int)blockIdx.x + (it / num_kb) * (int)gridDim.x) * ROWS_W; };
      auto k_of = [&](int it) { return (kb_begin + it % num_kb) * BK; };
      // W does not depend on the kernel before this one: the ring is filled with W tiles first,
      // then the kernel waits for its predecessor and sends the matching slices of A after them
      // W is read once per call and is far larger than the L2 over a step: its lines leave first
      const uint64_t once = l2_policy_evict_first();
      for (int it = 0; it < first; ++it) {
        mbar_expect_tx(&full_bar[it], C::STAGE_BYTES);
        tma_load_2d_hint(smem + it * C::STAGE_BYTES, &map_w, &full_bar[it], k_of(it), w_row(it), once);
      }
      STAMP(10);  // the ring's first tiles of W are requested
      pdl_wait();
      STAMP(1);  // the predecessor is complete
      for (int it = 0; it < first; ++it)
        tma_load_2d(smem + it * C::STAGE_BYTES + W_BYTES, &map_x, &full_bar[it], k_of(it), 0);
      for (int it = first; it < total; ++it) {
        const int s = it % C::STAGES;
        const uint32_t phase = (it / C::STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], phase ^ 1)) {
          failed = 1;
          break;
        }
        mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
        unsigned char* dst = smem + s * C::STAGE_BYTES;
        tma_load_2d_hint(dst, &map_w, &full_bar[s], k_of(it), w_row(it), once);
        tma_load_2d(dst + W_BYTES, &map_x, &full_bar[s], k_of(it), 0);
      }
      STAMP(7);  // the last tile of W is requested
      if (a.late_trigger) pdl_launch_dependents();
    }
  } else if (warp <= C::ISSUERS) {
    if (lane == 0) {
      // issuer j owns the k steps j, j + ISSUERS, ... of every k block and the partial accumulator j
      const int j = warp - 1;
      const uint32_t idesc = umma_idesc(ROWS_W, NB);
      int it = 0, local = 0;
      for (int nb = blockIdx.x; nb < n_blocks && !failed; nb += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!mbar_wait(&accum_empty[buf], ((local >> 1) & 1) ^ 1)) {
          failed = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * C::ACC_COLS + j * NB);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t phase = (it / C::STAGES) & 1;
          if (!mbar_wait(&full_bar[s], phase)) {
            failed = 1;
            break;
          }
          tc_fence_after();
          if (it == 0 && j == 0) STAMP(2);  // the first stage (W tile and slice of A) has landed
          const uint32_t w_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t x_addr = w_addr + W_BYTES;
          static_assert(BK / UMMA_K % C::ISSUERS == 0, "every issuer takes part in every k block");
#pragma unroll
          for (int k = 0; k < BK / UMMA_K / C::ISSUERS; ++k) {
            const int step = j + k * C::ISSUERS;
            umma(tmem_d, umma_desc(w_addr + step * 32), umma_desc(x_addr + step * 32), idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[s]);
        }
        if (failed) break;
        umma_commit(&accum_full[buf]);
        if (j == 0) STAMP(3);  // the last product of a block is issued
      }
    }
  }

  // ---- epilogue.  Thread (quarter, lane) of the four epilogue warps owns W row 32 * quarter + lane of
  // the block (a warp reaches the 32 lanes of tensor memory that its index modulo 4 names).
  const int quarter = warp & 3;
  const int row = quarter * 32 + lane;
  const bool swiglu = a.epilogue == EPI_SWIGLU;
  // The scales of a norm whose gain is already in A: rsqrt(mean square + eps) of the rows of
  // norm_src, by the four epilogue warps (rows in turn, 16-byte loads, 32-bit sums) while the
  // products run.  Called after the wait on the predecessor, which wrote those rows.
  __shared__ float row_scale[NB];
  // rows first, first + step, ... below M: the epilogue warps take them in turn, two rows of a warp
  // in flight at a time; a row's sum is formed the same way whoever asks (lanes stride over its
  // 16-byte pieces, then a tree over the lanes)
  auto compute_row_scales = [&](int first, int step) {
    if (a.norm_src == nullptr) return;
    const int pieces = a.K / 8;
    for (int m0 = first + (warp - C::FIRST_EPI_WARP) * step; m0 < a.M; m0 += 8 * step) {
      const int m1 = m0 + 4 * step;
      const uint4* src0 = reinterpret_cast<const uint4*>(a.norm_src + (size_t)m0 * a.ld_src);
      const uint4* src1 = reinterpret_cast<const uint4*>(a.norm_src + (size_t)(m1 < a.M ? m1 : m0) * a.ld_src);
      float ss0 = 0.f, ss1 = 0.f;
      for (int g0 = lane; g0 < pieces; g0 += 32 * 4) {
        uint4 u0[4], u1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int g = g0 + 32 * i;
          u0[i] = g < pieces ? src0[g] : make_uint4(0, 0, 0, 0);
          u1[i] = (g < pieces && m1 < a.M) ? src1[g] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ss0 += square_sum8(u0[i]);
          ss1 += square_sum8(u1[i]);
        }
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, sft);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, sft);
      }
      if (lane == 0) {
        row_scale[m0] = rsqrtf(ss0 / (float)a.K + a.norm_eps);
        if (m1 < a.M) row_scale[m1] = rsqrtf(ss1 / (float)a.K + a.norm_eps);
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
  };
  // The same for the rows a CTA of a cluster finishes (rank, rank + splits, ...): here the factors
  // are wanted soon after the wait, so all 128 threads share each row and eight to sixteen loads of
  // a thread are in flight: a CTA's whole share over 8 ranks at once (2, 4 or 8 rows), four pieces
  // of a row per thread (K up to 4096 in one trip to the L2), two at 64 rows of A.
  constexpr int OWN = NB == 16 ? 2 : NB == 32 ? 4 : 8, PIECES = NB == 64 ? 2 : 4;
  __shared__ float row_part[4][OWN];
  auto compute_own_row_scales = [&](int first, int step) {
    if (a.norm_src == nullptr) return;
    const int pieces = a.K / 8;
    const int t = (int)threadIdx.x - 32 * C::FIRST_EPI_WARP, w = t >> 5;
    for (int base = first; base < a.M; base += OWN * step) {
      float ss[OWN];
#pragma unroll
      for (int r = 0; r < OWN; ++r) ss[r] = 0.f;
      for (int g0 = t; g0 < pieces; g0 += 128 * PIECES) {
        uint4 u[OWN][PIECES];
#pragma unroll
        for (int r = 0; r < OWN; ++r) {
          const int m = base + r * step;
          const uint4* src = reinterpret_cast<const uint4*>(a.norm_src + (size_t)(m < a.M ? m : base) * a.ld_src);
#pragma unroll
          for (int i = 0; i < PIECES; ++i) {
            const int g = g0 + 128 * i;
            u[r][i] = (g < pieces && m < a.M) ? src[g] : make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int r = 0; r < OWN; ++r)
#pragma unroll
          for (int i = 0; i < PIECES; ++i) ss[r] += square_sum8(u[r][i]);
      }
#pragma unroll
      for (int r = 0; r < OWN; ++r) {
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], sft);
        if (lane == 0) row_part[w][r] = ss[r];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (t < OWN) {
        const int m = base + t * step;
        const float sum = ((row_part[0][t] + row_part[1][t]) + row_part[2][t]) + row_part[3][t];
        if (m < a.M) row_scale[m] = rsqrtf(sum / (float)a.K + a.norm_eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the factors are visible, the partial sums free again
    }
  };
  if (splits == 1) {
    if (warp >= C::FIRST_EPI_WARP) {
      pdl_wait();  // the residual comes from earlier kernels, and C may still be read by them
      if constexpr (NB <= 32) compute_row_scales(0, 1);
      else compute_own_row_scales(0, 1);  // many rows: more loads in flight
      int local = 0;
      for (int nb = blockIdx.x; nb < n_blocks; nb += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&accum_full[buf], (local >> 1) & 1))) {
          failed = 1;
          break;
        }
        tc_fence_after();
        if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(4);  // an accumulator is complete (the last one stays)
        // the accumulator in windows of WIN columns (rows h0 .. h0 + WIN - 1 of A); one window up to 64 rows
        constexpr int WIN = C::WINDOW;
        for (int h0 = 0; h0 < NB && h0 < a.M; h0 += WIN) {
        uint32_t v[WIN];
        load_accumulator<WIN, C::PARTS>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * C::ACC_COLS + h0), NB, v);
        if (h0 + WIN >= NB || h0 + WIN >= a.M) {  // the last window: the accumulator is free again
          tc_fence_before();
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&accum_empty[buf])) : "memory");
          if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(5);  // the accumulator is in registers
        }
        if (a.vec4 && !swiglu && a.residual == nullptr) {
          // Sixteen columns (rows of A) at a time go through shared memory and come back turned
          // around: a lane then holds four W rows of one row of A, the loop over the rows is rolled
          // (its instructions are fetched once) and a store carries four outputs.  (The output head
          // at 64 rows: 5.9 -> 1.9 us from the last accumulator to the last store.  The SwiGLU
          // epilogue written this way measured no faster than the form below, which pairs rows.)
          float* stage = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES) + (warp - C::FIRST_EPI_WARP) * 512;
          const int sub = lane >> 3, l8 = lane & 7;
          const int n4 = nb * ROWS_W + quarter * 32 + 4 * l8;
          float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), gain4 = bias4;
          if (n4 < a.N) {
            if (a.bias) bias4 = load4(a.bias + n4);
            if (a.C2) gain4 = load4(a.gain2 + n4);
          }
#pragma unroll
          for (int c0 = 0; c0 < WIN; c0 += 16) {
            if (h0 + c0 >= a.M) break;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 16; ++j) stage[j * 32 + lane] = __uint_as_float(v[c0 + j]);
            __syncwarp();
#pragma unroll 1
            for (int it = 0; it < 4; ++it) {
              const int m = h0 + c0 + 4 * it + sub;
              float4 val = *reinterpret_cast<const float4*>(stage + (4 * it + sub) * 32 + 4 * l8);
              if (a.norm_src) {
                const float scale = row_scale[m];
                val.x *= scale, val.y *= scale, val.z *= scale, val.w *= scale;
              }
              if (m < a.M && n4 < a.N) {
                val.x += bias4.x, val.y += bias4.y, val.z += bias4.z, val.w += bias4.w;
                store4(reinterpret_cast<TOut*>(a.C) + (size_t)m * a.ldc + n4, val);
                if (a.C2) {
                  const float4 out = rounded4<TOut>(val);
                  store4(reinterpret_cast<TOut*>(a.C2) + (size_t)m * a.ldc2 + n4,
                         make_float4(out.x * gain4.x, out.y * gain4.y, out.z * gain4.z, out.w * gain4.w));
                }
              }
            }
          }
          continue;  // the next window
        }
        // (SwiGLU, a residual, or rows or pointers that do not allow that: one output per thread and row)
        if (a.norm_src) {
#pragma unroll
          for (int m = 0; m < WIN; ++m)
            if (h0 + m < a.M) v[m] = __float_as_uint(__uint_as_float(v[m]) * row_scale[h0 + m]);
        }
        const int n = nb * ROWS_W + row;
        if (swiglu) {
          // lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same 16 outputs.  Two rows
          // of A at a time: the low lanes finish the first (they get its up values), the high
          // lanes the second (they get its gate values), so every lane computes.
          const bool low = lane < 16;
          const int col = ((n - lane) >> 1) + (lane & 15);
          const bool n_ok = n - lane < a.N;  // N is a multiple of 32: the block of 32 rows is whole
#pragma unroll
          for (int m0 = 0; m0 < WIN; m0 += 2) {
            const float x0 = __uint_as_float(v[m0]), x1 = __uint_as_float(v[m0 + 1]);
            const float other = __shfl_xor_sync(0xffffffffu, low ? x1 : x0, 16);
            const float gate = low ? x0 : other, up = low ? other : x1;
            const int m = h0 + (low ? m0 : m0 + 1);
            if (m < a.M && n_ok)
              reinterpret_cast<TOut*>(a.C)[(size_t)m * a.ldc + col] = from_f32<TOut>(silu_times(gate, up));
          }
        } else {
#pragma unroll
          for (int m = 0; m < WIN; ++m)
            if (h0 + m < a.M && n < a.N) finish<TOut>(a, __uint_as_float(v[m]), h0 + m, n);
        }
        }  // windows
        if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(9);  // the block's stores are issued
      }
    }
    __syncthreads();
  } else {
    // One block per CTA; the cluster adds the partial tiles.  This part runs once per CTA, so what
    // it costs is the instructions it fetches and the trips it waits for, and it is written for
    // few of both.  Every thread puts its accumulators (one W row, all rows of A) into the drained
    // ring, [row of A][128]; a warp sends whole rows of A, 16 bytes a lane, to the CTA that
    // finishes them (row m to rank m % splits) by remote stores that count their bytes on the
    // receiver's barrier; a CTA waits for the bytes due in its inbox and a warp finishes whole
    // rows, four outputs a lane.  The loops over rows are rolled.  Up to 16 rows of A the inbox
    // has room of its own behind the ring, so nobody waits for the cluster (the barrier whose first
    // half was passed at the start only says that every CTA is running); with more rows it is a
    // second part of the ring, and one cluster barrier says that every CTA is through with its ring.
    // (Measured on the whole decode step of the 1.5B shape.  64 rows: partial tiles read from every
    // rank between two cluster barriers 1.89 ms; this form 1.79 ms; the same with one bulk copy per
    // row and a second barrier that keeps the tiles in place 1.80 ms; with one bulk copy per rank
    // from a tile ordered by rank 2.00 ms, its unrolled stores with computed addresses being the
    // cost.  8 rows: every thread sending its own 4-byte values, unrolled, 1.000 ms; this form
    // 0.988 ms; 1 row 0.989 -> 0.949 ms.)
    const int rows_per = (a.M + splits - 1) / splits;
    float* tile = reinterpret_cast<float*>(smem);                    // [row of A][128]
    // [source rank][rows per CTA][128]: behind the ring where there is room for it (up to 16 rows)
    float* inbox = C::PUSH ? reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES) : tile + NB * ROWS_W;
    if constexpr (C::PUSH) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // second half of the start barrier
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int rows_own = rank < a.M ? (a.M - rank + splits - 1) / splits : 0;
    const int ew = warp - C::FIRST_EPI_WARP;                          // 0..3 in the epilogue warps
    const int n4 = blockIdx.x * ROWS_W + 4 * lane;                    // this lane's four outputs of a row
    const bool n_ok = n4 < a.N;                                       // N is a multiple of 4 here
    // bias, and the residual of the first rows this warp finishes (its share at 64 or 128 rows over 8
    // ranks), are asked for while the products still run
    constexpr int RES = NB <= 64 ? 2 : 4;  // rows of a warp's share whose residual is asked for ahead
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), gain4 = bias4, res4[RES];
    if (warp >= C::FIRST_EPI_WARP) {
      pdl_wait();  // the residual comes from earlier kernels, and C may still be read by them
      if (!swiglu && n_ok) {
        if (a.bias) bias4 = load4(a.bias + n4);
        if (a.C2) gain4 = load4(a.gain2 + n4);
      }
#pragma unroll
      for (int i = 0; i < RES; ++i) {
        const int m = rank + (ew + 4 * i) * splits;
        res4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!swiglu && n_ok && a.residual && m < a.M)
          res4[i] = load4(reinterpret_cast<const TOut*>(a.residual) + (size_t)m * a.ldr + n4);
      }
      compute_own_row_scales(rank, splits);
      if (!__all_sync(0xffffffffu, mbar_wait(&accum_full[0], 0))) failed = 1;
      tc_fence_after();
      if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(4);  // the accumulator is complete
      for (int h0 = 0; h0 < NB && h0 < a.M; h0 += C::WINDOW) {
        uint32_t v[C::WINDOW];
        load_accumulator<C::WINDOW, C::PARTS>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)h0, NB, v);
#pragma unroll
        for (int m = 0; m < C::WINDOW; ++m) tile[(h0 + m) * ROWS_W + row] = __uint_as_float(v[m]);
      }
    }
    if constexpr (C::PUSH) {
      // the inbox is nobody's ring: only this CTA's epilogue warps meet, over the tile
      if (warp >= C::FIRST_EPI_WARP) asm volatile("bar.sync 1, 128;" ::: "memory");
    } else {
      tc_fence_before();
      __syncthreads();
      cluster.sync();  // every CTA's products are done: the rings are free, the tiles in place
    }
    if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(11);
    if (warp >= C::FIRST_EPI_WARP) {
      if (!failed) {
        // a warp sends whole rows of A, 16 bytes a lane: row m to rank m % splits, slot m / splits
#pragma unroll 1
        for (int m = ew; m < a.M; m += 4) {
          const uint32_t owner = (uint32_t)(m % splits);
          const int slot = m / splits;
          const float4 val = reinterpret_cast<const float4*>(tile + m * ROWS_W)[lane];
          const uint32_t dst = mapa_u32(smem_u32(inbox + (rank * rows_per + slot) * ROWS_W + 4 * lane), owner);
          st_async_v4(dst, val, mapa_u32(smem_u32(&inbox_bar), owner));
        }
      }
      if (threadIdx.x == 32 * C::FIRST_EPI_WARP) mbar_expect_tx(&inbox_bar, (uint32_t)(splits * rows_own * ROWS_W * 4));
      if (!__all_sync(0xffffffffu, mbar_wait(&inbox_bar, 0))) failed = 1;
      if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(5);  // every rank's rows have arrived
      if (!failed) {
#pragma unroll 1
        for (int slot = ew, i = 0; slot < rows_own; slot += 4, ++i) {
          const int m = rank + slot * splits;
          float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int sp = 0; sp < MAX_SPLITS; ++sp) {  // in rank order
            if (sp < splits) {
              const float4 part = reinterpret_cast<const float4*>(inbox + (sp * rows_per + slot) * ROWS_W)[lane];
              total.x += part.x, total.y += part.y, total.z += part.z, total.w += part.w;
            }
          }
          if (a.norm_src) {
            const float scale = row_scale[m];
            total.x *= scale, total.y *= scale, total.z *= scale, total.w *= scale;
          }
          if (swiglu) {
            // a lane holds four W rows; of every 32 rows the first 16 are gates, the other 16 the up
            // rows of the same outputs: lanes 0..3 of eight pair with lanes 4..7
            float4 up;
            up.x = __shfl_down_sync(0xffffffffu, total.x, 4);
            up.y = __shfl_down_sync(0xffffffffu, total.y, 4);
            up.z = __shfl_down_sync(0xffffffffu, total.z, 4);
            up.w = __shfl_down_sync(0xffffffffu, total.w, 4);
            if ((lane & 4) == 0 && n4 + 16 < a.N) {
              const int col = ((blockIdx.x * ROWS_W + (lane >> 3) * 32) >> 1) + 4 * (lane & 3);
              store4(reinterpret_cast<TOut*>(a.C) + (size_t)m * a.ldc + col,
                     make_float4(silu_times(total.x, up.x), silu_times(total.y, up.y), silu_times(total.z, up.z),
                                 silu_times(total.w, up.w)));
            }
          } else if (n_ok) {
            float4 res = res4[0];
#pragma unroll
            for (int q = 1; q < RES; ++q)
              if (i == q) res = res4[q];
            if (i >= RES && a.residual) res = load4(reinterpret_cast<const TOut*>(a.residual) + (size_t)m * a.ldr + n4);
            // the same order of sums as finish(): bias, then residual
            total.x = (total.x + bias4.x) + res.x, total.y = (total.y + bias4.y) + res.y;
            total.z = (total.z + bias4.z) + res.z, total.w = (total.w + bias4.w) + res.w;
            store4(reinterpret_cast<TOut*>(a.C) + (size_t)m * a.ldc + n4, total);
            if (a.C2) {
              const float4 out = rounded4<TOut>(total);
              store4(reinterpret_cast<TOut*>(a.C2) + (size_t)m * a.ldc2 + n4,
                     make_float4(out.x * gain4.x, out.y * gain4.y, out.z * gain4.z, out.w * gain4.w));
            }
          }
        }
      }
      if (threadIdx.x == 32 * C::FIRST_EPI_WARP) STAMP(9);  // this CTA's rows are stored
    }
  }

  // every warp is through with the tensor memory before it is given back
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) STAMP(6);  // every store of this CTA is issued
  if (failed) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_WAIT_LIMIT);
    // let copies that are still on their way land before the shared memory goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

template <int NB, typename TOut>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const Args& a, int n_blocks, int splits, int num_sms,
           int* err, cudaStream_t stream) {
  using C = Cfg<NB>;
  const size_t smem = (size_t)C::STAGES * C::STAGE_BYTES + 1024 + C::INBOX_BYTES;
  auto kernel = gemm_stream_kernel<NB, TOut>;
  static bool configured = false;
  if (!configured) {
    DSP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  const int resident = C::MIN_CTAS * num_sms;  // without a split the CTAs walk over the blocks of W
  cfg.gridDim = dim3(splits > 1 ? n_blocks : (n_blocks < resident ? n_blocks : resident), splits, 1);
  cfg.blockDim = dim3(C::THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  DSP_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, a, err));
  return 0;
}
}  // namespace

#ifdef DSP_STAMPS
namespace {
long g_stamp_cursor = -1;  // -1: off
long g_stamp_log[4096][4];  // per launch: first slot, CTAs, N, K
int g_stamp_launches = 0;
long stamp_next_base(long ctas, int N, int K) {
  if (g_stamp_cursor < 0 || g_stamp_cursor + ctas * 12 > (1 << 21) || g_stamp_launches >= 4096) return -1;
  const long base = g_stamp_cursor;
  g_stamp_cursor += ctas * 12;
  g_stamp_log[g_stamp_launches][0] = base;
  g_stamp_log[g_stamp_launches][1] = ctas;
  g_stamp_log[g_stamp_launches][2] = N;
  g_stamp_log[g_stamp_launches][3] = K;
  ++g_stamp_launches;
  return base;
}
}  // namespace
// The launches recorded so far: four numbers each (first slot, CTAs, N, K); returns how many.
extern "C" int dsp_gemm_stream_stamps_log(long* out, int max_launches) {
  const int n = g_stamp_launches < max_launches ? g_stamp_launches : max_launches;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < 4; ++j) out[i * 4 + j] = g_stamp_log[i][j];
  return n;
}
// Starts (on = 1, from slot 0) or stops recording; returns the slots used so far.
extern "C" long dsp_gemm_stream_stamps_control(int on) {
  const long used = g_stamp_cursor < 0 ? 0 : g_stamp_cursor;
  g_stamp_cursor = on ? 0 : -1;
  if (on) g_stamp_launches = 0;
  return used;
}
extern "C" int dsp_gemm_stream_stamps_read(unsigned long long* out, long n) {
  DSP_CUDA(cudaMemcpyFromSymbol(out, g_stamps, (size_t)n * sizeof(unsigned long long)));
  return 0;
}
#endif

// epilogue: 0 plain (bias, residual allowed); 1 SwiGLU over W rows alternating in blocks of 16
// (C is [M, N/2]; no bias, no residual).  target_ctas: resident CTA slots the launch may fill by
// splitting K (0: one per SM).  late_trigger_bytes: a product that streams at least this many bytes
// of W lets the next kernel start only when its own last tile is on its way (what the next kernels
// request before their wait would otherwise compete with a long stream); shorter products let it
// start at once; 0 or less: always at once.
// norm_src (bfloat16 rows of K values, row stride ld_src) and norm_eps: the rows of the product are
// multiplied by rsqrt(mean(norm_src[m]^2) + norm_eps) before bias and residual (A holds those rows
// times a norm's gain: together that is the norm in front of the product).  gain2 (bfloat16 [N])
// and C2 (the output's type, row stride ldc2): also stores the rounded output times gain2, with
// the plain epilogue.
extern "C" int dsp_gemm_stream(const void* A, long lda, const void* W, const void* bias, const void* residual,
                               long ldr, void* C, long ldc, int M, int N, int K, int out_dtype, int target_ctas,
                               int epilogue, long late_trigger_bytes, const void* norm_src, long ld_src,
                               float norm_eps, const void* gain2, void* C2, long ldc2, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DSP_REQUIRE(norm_src == nullptr || (ld_src % 8 == 0 && ((uintptr_t)norm_src % 16) == 0),
              "dsp_gemm_stream: the rows under the norm must be 16-byte aligned (row stride %ld)", ld_src);
  DSP_REQUIRE(C2 == nullptr || (gain2 != nullptr && epilogue == EPI_PLAIN),
              "dsp_gemm_stream: the scaled second output needs a gain and the plain epilogue");
  DSP_REQUIRE(M <= 128, "dsp_gemm_stream: M=%d above 128 rows", M);
  DSP_REQUIRE(M <= 64 || (norm_src == nullptr && C2 == nullptr),
              "dsp_gemm_stream: a norm split over two products takes at most 64 rows, got %d", M);
  DSP_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0, "dsp_gemm_stream: K=%d and the row stride must be multiples of 8", K);
  DSP_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0, "dsp_gemm_stream: operands must be 16-byte aligned");
  DSP_REQUIRE(out_dtype == DSP_BF16 || out_dtype == DSP_F32, "dsp_gemm_stream: unknown output dtype %d", out_dtype);
  DSP_REQUIRE(epilogue == EPI_PLAIN || (N % 32 == 0 && bias == nullptr && residual == nullptr),
              "dsp_gemm_stream: the SwiGLU epilogue needs N in whole blocks of 32 and no bias or residual");
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_gemm_stream: no device error word");
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    DSP_CUDA(cudaGetDevice(&dev));
    DSP_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int nb_rows = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  CUtensorMap map_w, map_x;
  DSP_REQUIRE(make_map(&map_w, W, N, K, K, ROWS_W), "dsp_gemm_stream: cannot encode the tensor map of W");
  DSP_REQUIRE(make_map(&map_x, A, M, K, lda, nb_rows), "dsp_gemm_stream: cannot encode the tensor map of A");
  const int n_blocks = (N + ROWS_W - 1) / ROWS_W;
  const int kb_total = (K + BK - 1) / BK;
  if (target_ctas <= 0) target_ctas = num_sms;
  int splits = target_ctas / n_blocks;
  if (splits < 1) splits = 1;
  if (splits > MAX_SPLITS) splits = MAX_SPLITS;
  if (splits > kb_total) splits = kb_total;
  // the epilogues move four outputs at a time where rows and pointers allow 16-byte (32-bit output)
  // or 8-byte accesses; where they do not, K is not split and every thread stores single outputs
  const uintptr_t mask = out_dtype == DSP_F32 ? 15 : 7;
  const bool vec_ok = N % 4 == 0 && ldc % 4 == 0 && ((uintptr_t)C & mask) == 0 &&
                      (residual == nullptr || (ldr % 4 == 0 && ((uintptr_t)residual & mask) == 0)) &&
                      (bias == nullptr || ((uintptr_t)bias & 7) == 0) &&
                      (C2 == nullptr || (ldc2 % 4 == 0 && ((uintptr_t)C2 & mask) == 0 && ((uintptr_t)gain2 & 7) == 0));
  if (!vec_ok) splits = 1;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per_split - 1) / kb_per_split;
  Args a;
  a.stamp_base = -1;
#ifdef DSP_STAMPS
  a.stamp_base = stamp_next_base(splits > 1 ? (long)n_blocks * splits : (n_blocks < (nb_rows > 64 ? 1 : 2) * num_sms ? n_blocks : (nb_rows > 64 ? 1 : 2) * num_sms), N, K);
#endif
  a.bias = (const bf16*)bias;
  a.residual = residual;
  a.ldr = ldr;
  a.C = C;
  a.ldc = ldc;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kb_per_split = kb_per_split;
  a.epilogue = epilogue;
  a.late_trigger = (late_trigger_bytes > 0 && (long)N * K * 2 >= late_trigger_bytes) ? 1 : 0;
  a.vec4 = vec_ok ? 1 : 0;
  a.norm_src = (const bf16*)norm_src;
  a.ld_src = ld_src;
  a.norm_eps = norm_eps;
  a.gain2 = (const bf16*)gain2;
  a.C2 = C2;
  a.ldc2 = ldc2;
  if (out_dtype == DSP_BF16) {
    if (nb_rows == 16) return launch<16, bf16>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
    if (nb_rows == 32) return launch<32, bf16>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
    if (nb_rows == 64) return launch<64, bf16>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
    return launch<128, bf16>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
  }
  if (nb_rows == 16) return launch<16, float>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
  if (nb_rows == 32) return launch<32, float>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
  if (nb_rows == 64) return launch<64, float>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
  return launch<128, float>(map_w, map_x, a, n_blocks, splits, num_sms, err, stream);
}
