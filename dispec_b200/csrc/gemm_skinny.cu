// C[M,N] = A[M,K] * W[N,K]^T (+ bias) (+ residual) for M <= 64 rows, bfloat16 in, 32-bit
// accumulation: the matrix product of decoding, bound by streaming W once from HBM.
//
// Roles are swapped for the tensor cores: W is the 16-row operand of mma.m16n8k16, the few rows
// of A are its 8-column operand.  Each warp streams 32 rows of W straight from global memory
// into registers (16-byte loads, eight 32-wide k blocks in flight) and takes A from shared
// memory, where the CTA stages it in 256-wide k chunks (cp.async, two stages).  The k index
// inside a 32-wide block is permuted identically for both operands so that every thread's
// 16-byte load lands in its own fragments without a shuffle.
//
// Split-K: grid.y CTAs share the K range of one 128-row block of W; each writes its partial
// tile to scratch memory, and the last one to arrive (a counter per block) adds the partials in
// split order, so the result is deterministic, then applies bias and residual and resets the
// counter.  Calls that overlap in time on the device must not share scratch and counters.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int ROWS_PER_WARP = 32;
constexpr int BLOCK_N = WARPS * ROWS_PER_WARP;  // 128 rows of W per CTA
constexpr int KC = 256;                         // k chunk staged in shared memory
constexpr int KB_PER_CHUNK = KC / 32;
constexpr int A_STRIDE = KC * 2 + 64;           // bytes; 16-byte units = 4 mod 8: conflict-free

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// MT: number of 8-row tiles of A (rows padded to 8 * MT)
template <int MT, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const bf16* __restrict__ A, long lda, const bf16* __restrict__ W,
                   const bf16* __restrict__ bias, const TOut* __restrict__ residual, long ldr,
                   TOut* __restrict__ C, long ldc, int M, int N, int K, int chunks_per_split,
                   float* __restrict__ scratch, int* __restrict__ counters) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int nb = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int n_warp = nb * BLOCK_N + warp * ROWS_PER_WARP;
  const int MP = MT * 8;

  const int chunk_begin = split * chunks_per_split;
  const int total_chunks = (K + KC - 1) / KC;
  const int chunk_end = min(total_chunks, chunk_begin + chunks_per_split);

  float acc[2][MT][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[s][mt][r] = 0.f;

  // rows of W this lane reads (clamped: rows beyond N are computed but never stored)
  const bf16* wrow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = min(n_warp + g + 8 * i, N - 1);
    wrow[i] = W + (size_t)n * K;
  }

  unsigned char* stage[2] = {smem, smem + MP * A_STRIDE};
  auto load_stage = [&](int chunk, int buf) {
    const int k0 = chunk * KC;
    // MP rows x 32 sixteen-byte pieces
    for (int i = tid; i < MP * 32; i += THREADS) {
      const int row = i >> 5, piece = i & 31;
      const int k = k0 + piece * 8;
      const bool valid = row < M && k < K;
      const bf16* src = valid ? A + (size_t)row * lda + k : A;
      cp_async16(stage[buf] + row * A_STRIDE + piece * 16, src, valid);
    }
    cp_async_commit();
  };

  if (chunk_begin < chunk_end) load_stage(chunk_begin, 0);
  for (int chunk = chunk_begin; chunk < chunk_end; ++chunk) {
    const int buf = (chunk - chunk_begin) & 1;
    if (chunk + 1 < chunk_end) {
      load_stage(chunk + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int k0 = chunk * KC;
    const unsigned char* xs = stage[buf];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      // four 32-wide k blocks at a time: 16 loads of 16 bytes in flight per lane
      uint4 w[4][4];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        const int k = k0 + (half * 4 + kb) * 32 + c * 8;
        const bool valid = k < K;
        const int ks = valid ? k : 0;  // load unconditionally, discard afterwards
#pragma unroll
        for (int i = 0; i < 4; ++i) w[kb][i] = ldg_stream(wrow[i] + ks);
        if (!valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) w[kb][i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        const int piece = (half * 4 + kb) * 4 + c;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 x = *reinterpret_cast<const uint4*>(xs + (mt * 8 + g) * A_STRIDE + piece * 16);
          // strip 0: rows g, g+8; strip 1: rows g+16, g+24
          mma_bf16(acc[0][mt], w[kb][0].x, w[kb][1].x, w[kb][0].y, w[kb][1].y, x.x, x.y);
          mma_bf16(acc[0][mt], w[kb][0].z, w[kb][1].z, w[kb][0].w, w[kb][1].w, x.z, x.w);
          mma_bf16(acc[1][mt], w[kb][2].x, w[kb][3].x, w[kb][2].y, w[kb][3].y, x.x, x.y);
          mma_bf16(acc[1][mt], w[kb][2].z, w[kb][3].z, w[kb][2].w, w[kb][3].w, x.z, x.w);
        }
      }
    }
    __syncthreads();
  }

  constexpr int R = 2 * MT * 4;  // accumulators per thread
  if (splits > 1) {
    float* mine = scratch + ((size_t)(split * gridDim.x + nb) * R) * THREADS;
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 4; ++r) mine[((s * MT + mt) * 4 + r) * THREADS + tid] = acc[s][mt][r];
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&counters[nb], 1) == splits - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float total = 0.f;
          for (int sp = 0; sp < splits; ++sp)
            total += __ldcg(scratch + ((size_t)(sp * gridDim.x + nb) * R + ((s * MT + mt) * 4 + r)) * THREADS + tid);
          acc[s][mt][r] = total;
        }
    if (tid == 0) counters[nb] = 0;
  }

  // accumulator (s, mt, r): W row n = n_warp + 16 s + g + 8 (r / 2), A row m = 8 mt + 2 c + (r & 1)
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n = n_warp + 16 * s + g + 8 * (r >> 1);
        const int m = 8 * mt + 2 * c + (r & 1);
        if (n < N && m < M) {
          float v = acc[s][mt][r];
          if (bias) v += __bfloat162float(bias[n]);
          if (residual) v += to_f32(residual[(size_t)m * ldr + n]);
          C[(size_t)m * ldc + n] = from_f32<TOut>(v);
        }
      }
}

template <int MT, typename TOut>
int launch(const void* A, long lda, const void* W, const void* bias, const void* residual, long ldr,
           void* C, long ldc, int M, int N, int K, int splits, int chunks_per_split, float* scratch,
           int* counters, cudaStream_t stream) {
  const size_t smem = 2 * (size_t)(MT * 8) * A_STRIDE;
  auto kernel = gemm_skinny_kernel<MT, TOut>;
  DSP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((N + BLOCK_N - 1) / BLOCK_N, splits);
  kernel<<<grid, THREADS, smem, stream>>>((const bf16*)A, lda, (const bf16*)W, (const bf16*)bias,
                                          (const TOut*)residual, ldr, (TOut*)C, ldc, M, N, K,
                                          chunks_per_split, scratch, counters);
  DSP_CHECK_LAUNCH("dsp_gemm_skinny");
  return 0;
}

template <typename TOut>
int dispatch(const void* A, long lda, const void* W, const void* bias, const void* residual, long ldr,
             void* C, long ldc, int M, int N, int K, int splits, int cps, float* scratch,
             int* counters, cudaStream_t stream) {
  if (M <= 8) return launch<1, TOut>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
  if (M <= 16) return launch<2, TOut>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
  if (M <= 32) return launch<4, TOut>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
  return launch<8, TOut>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
}
}  // namespace

// Number of K splits the launch below will use (the caller sizes scratch with it).
extern "C" int dsp_gemm_skinny_splits(int N, int K, int target_ctas) {
  const int n_blocks = (N + BLOCK_N - 1) / BLOCK_N;
  const int chunks = (K + KC - 1) / KC;
  int splits = target_ctas / n_blocks;
  if (splits < 1) splits = 1;
  if (splits > chunks) splits = chunks;
  const int cps = (chunks + splits - 1) / splits;
  return (chunks + cps - 1) / cps;
}

// scratch: floats, at least splits * ceil(N/128) * 128 * 8 * ceil8(M) when splits > 1.
// counters: ceil(N/128) ints, zero before the first call (the kernel leaves them zero).
extern "C" int dsp_gemm_skinny(const void* A, long lda, const void* W, const void* bias,
                               const void* residual, long ldr, void* C, long ldc, int M, int N,
                               int K, int out_dtype, int target_ctas, float* scratch,
                               long scratch_floats, int* counters, int num_counters,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DSP_REQUIRE(M <= 64, "dsp_gemm_skinny: M=%d above 64 rows", M);
  DSP_REQUIRE(K > 0 && K % 8 == 0, "dsp_gemm_skinny: K=%d must be a positive multiple of 8", K);
  DSP_REQUIRE(lda % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0,
              "dsp_gemm_skinny: operands must be 16-byte aligned with a row stride multiple of 8");
  const int n_blocks = (N + BLOCK_N - 1) / BLOCK_N;
  const int chunks = (K + KC - 1) / KC;
  int splits = dsp_gemm_skinny_splits(N, K, target_ctas);
  const int mt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
  if (splits > 1) {
    const long need = (long)splits * n_blocks * THREADS * 8 * mt;
    if (scratch == nullptr || counters == nullptr || need > scratch_floats || n_blocks > num_counters)
      splits = 1;  // no room to split: still correct, only slower
  }
  const int cps = (chunks + splits - 1) / splits;
  splits = (chunks + cps - 1) / cps;
  DSP_REQUIRE(splits <= 65535, "dsp_gemm_skinny: too many splits");
  if (out_dtype == DSP_BF16)
    return dispatch<bf16>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
  if (out_dtype == DSP_F32)
    return dispatch<float>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, splits, cps, scratch, counters, stream);
  DSP_REQUIRE(false, "dsp_gemm_skinny: unknown output dtype %d", out_dtype);
}
