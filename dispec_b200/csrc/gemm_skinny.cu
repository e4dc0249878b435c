// C[M,N] = op(A)[M,K] * W[N,K]^T (+ bias) (+ residual) for M <= 64 rows, bfloat16 in, 32-bit
// accumulation: the matrix product of decoding, bound by streaming W once from HBM.
//
// Roles are swapped for the tensor cores: W is the 16-row operand of mma.m16n8k16, the few rows
// of A are its 8-column operand.  Each warp streams 32 rows of W in groups of four 32-wide k
// blocks (16 pieces of 16 bytes per lane, 8 KB per warp).  The pieces travel by cp.async into a
// ring in shared memory that is private to the lane that asked for them: the lane reads back
// exactly what it copied, so the ring needs no barrier, only cp.async.wait_group, and serves as a
// deep prefetch queue (five groups, 40 KB per warp, on their way at any time) that registers
// could not hold.  The k index inside a 32-wide block is permuted identically for both operands
// so that every lane's 16-byte piece lands in its own fragments without a shuffle.
//
// A comes from global memory directly for up to 16 rows (it stays in L1/L2), optionally
// transformed on the way in:
//   prologue 1: RMSNorm, a = round(gain[k] * round(x * rsqrt(mean(x^2) + eps))), the row
//               statistics recomputed by every CTA (a few KB of reads);
// Epilogue SwiGLU: W holds gate and up rows interleaved in blocks of 16 (16 gate rows, then the
// 16 up rows of the same outputs), so a warp's 32-row strip has both halves of 16 outputs and
// writes silu(gate) * up, [M, N/2], instead of the raw products.
// For 17..64 rows A is staged through shared memory in 256-wide k chunks (cp.async, two stages).
//
// Split-K: the CTAs that share one block of W rows form a thread-block cluster (up to 8); each
// leaves its partial tile in its own shared memory, and after a cluster barrier every CTA adds a
// share of the tile over all ranks in rank order (distributed shared memory), so the sum is
// deterministic and needs no global scratch.  Bias and residual are applied by the adding CTA.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {
constexpr int KC = 256;                // k chunk of the staged path
constexpr int A_STRIDE = KC * 2 + 64;  // bytes; in 16-byte units = 4 mod 8: conflict-free
constexpr int MAX_SPLITS = 8;          // portable cluster size

enum Prologue { PRO_NONE = 0, PRO_RMSNORM = 1 };
enum Epilogue { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

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
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

struct Args {
  const bf16* A;
  long lda;
  const bf16* W;
  const bf16* bias;
  const void* residual;
  long ldr;
  void* C;
  long ldc;
  int M, N, K;
  int groups_per_split;  // k range of one split, in groups of 128
  const bf16* gain;      // prologue 1
  float eps;
  int epilogue;
};

// eight bfloat16 values of one A fragment piece, transformed by the prologue
template <int PRO>
__device__ __forceinline__ uint4 load_a_piece(const Args& a, int row, int k, const float* rstd) {
  const bool valid = row < a.M && k < a.K;
  const int rs = valid ? row : 0, ks = valid ? k : 0;
  uint4 raw = ldg_cached(a.A + (size_t)rs * a.lda + ks);
  if (PRO == PRO_RMSNORM) {
    const uint4 graw = ldg_cached(a.gain + ks);
    const bf16* x = reinterpret_cast<const bf16*>(&raw);
    const bf16* gn = reinterpret_cast<const bf16*>(&graw);
    uint4 out;
    bf16* o = reinterpret_cast<bf16*>(&out);
    const float r = rstd[rs];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bf16 n = __float2bfloat16(__bfloat162float(x[j]) * r);
      o[j] = __float2bfloat16(__bfloat162float(gn[j]) * __bfloat162float(n));
    }
    raw = out;
  }
  if (!valid) raw = make_uint4(0u, 0u, 0u, 0u);
  return raw;
}

// MT: 8-row tiles of A.  WARPS: warps per CTA (32 rows of W each).  STAGED: A through shared memory.
template <int MT, int WARPS, bool STAGED, int PRO, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const Args a) {
  constexpr int THREADS = WARPS * 32;
  constexpr int R = 2 * MT * 4;  // accumulators per thread
  constexpr int STAGES = STAGED ? 3 : 6;
  constexpr int RING_BYTES = WARPS * STAGES * 8192;  // 8 KB per warp and stage
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float rstd[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int nb = blockIdx.x;
  const int splits = gridDim.y;
  const int split = blockIdx.y;
  const int n_warp = nb * (WARPS * 32) + warp * 32;
  const int MP = MT * 8;

  const int total_groups = (a.K + 127) / 128;
  const int group_begin = split * a.groups_per_split;
  const int group_end = min(total_groups, group_begin + a.groups_per_split);

  // rows of W this lane reads (clamped: rows beyond N are computed but never stored)
  const bf16* wrow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) wrow[i] = a.W + (size_t)min(n_warp + g + 8 * i, a.N - 1) * a.K;

  // the lane's slots of the ring: [stage][k block][row i][lane], 16 bytes each
  unsigned char* ring = smem + warp * (STAGES * 8192) + lane * 16;
  auto issue_w = [&](int group, int stage) {
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const int k = group * 128 + kb * 32 + c * 8;
      const bool valid = k < a.K;
      const int ks = valid ? k : 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        cp_async16(ring + ((stage * 4 + kb) * 4 + i) * 512, wrow[i] + ks, valid);
    }
  };
  auto read_w = [&](uint4 (&w)[4][4], int stage) {
#pragma unroll
    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[kb][i] = *reinterpret_cast<const uint4*>(ring + ((stage * 4 + kb) * 4 + i) * 512);
  };

  float acc[2][MT][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[s][mt][r] = 0.f;

  // the first groups are on their way before anything else happens
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (group_begin + st < group_end) issue_w(group_begin + st, st);
    cp_async_commit();
  }
  // weights do not depend on the kernel before this one; everything below does
  pdl_launch_dependents();
  pdl_wait();

  if (PRO == PRO_RMSNORM) {
    // row statistics over the whole of K, recomputed by every CTA: warp w takes rows w, w+WARPS, ..
    for (int row = warp; row < a.M; row += WARPS) {
      float ss = 0.f;
      for (int k = lane * 8; k < a.K; k += 256) {
        const uint4 raw = ldg_cached(a.A + (size_t)row * a.lda + k);
        const bf16* x = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __bfloat162float(x[j]);
          ss += v * v;
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) rstd[row] = rsqrtf(ss / (float)a.K + a.eps);
    }
    __syncthreads();
  }

  unsigned char* stage[2] = {smem + RING_BYTES, smem + RING_BYTES + MP * A_STRIDE};
  auto load_stage = [&](int chunk, int buf) {
    const int k0 = chunk * KC;
    for (int i = tid; i < MP * 32; i += THREADS) {
      const int row = i >> 5, piece = i & 31;
      const int k = k0 + piece * 8;
      const bool valid = row < a.M && k < a.K;
      const bf16* src = valid ? a.A + (size_t)row * a.lda + k : a.A;
      cp_async16(stage[buf] + row * A_STRIDE + piece * 16, src, valid);
    }
    cp_async_commit();
  };

  auto load_x = [&](uint4 (&x)[4][MT], int group) {
#pragma unroll
    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        x[kb][mt] = load_a_piece<PRO>(a, mt * 8 + g, group * 128 + kb * 32 + c * 8, rstd);
  };
  auto compute = [&](uint4 (&x)[4][MT], int group, int w_stage, const unsigned char* xs) {
    uint4 w[4][4];
    read_w(w, w_stage);
    if (STAGED) {
      const int piece0 = (group & 1) * 16 + c;  // two groups per 256-wide chunk
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          x[kb][mt] = *reinterpret_cast<const uint4*>(xs + (mt * 8 + g) * A_STRIDE + (piece0 + kb * 4) * 16);
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        // strip 0: rows g, g+8; strip 1: rows g+16, g+24
        mma_bf16(acc[0][mt], w[kb][0].x, w[kb][1].x, w[kb][0].y, w[kb][1].y, x[kb][mt].x, x[kb][mt].y);
        mma_bf16(acc[0][mt], w[kb][0].z, w[kb][1].z, w[kb][0].w, w[kb][1].w, x[kb][mt].z, x[kb][mt].w);
        mma_bf16(acc[1][mt], w[kb][2].x, w[kb][3].x, w[kb][2].y, w[kb][3].y, x[kb][mt].x, x[kb][mt].y);
        mma_bf16(acc[1][mt], w[kb][2].z, w[kb][3].z, w[kb][2].w, w[kb][3].w, x[kb][mt].z, x[kb][mt].w);
      }
  };

  if (!STAGED) {
    uint4 x_cur[4][MT], x_next[4][MT];
    if (group_begin < group_end) load_x(x_cur, group_begin);
    for (int gi = group_begin; gi < group_end; ++gi) {
      const int j = gi - group_begin;
      const int nxt = gi + STAGES - 1;
      if (nxt < group_end) issue_w(nxt, (j + STAGES - 1) % STAGES);
      cp_async_commit();
      if (gi + 1 < group_end) load_x(x_next, gi + 1);  // one group ahead, behind the L2 latency
      cp_async_wait<STAGES - 1>();                     // group gi has landed
      compute(x_cur, gi, j % STAGES, nullptr);
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) x_cur[kb][mt] = x_next[kb][mt];
    }
  } else {
    // group_begin is even (a split starts on a chunk boundary): chunk = group / 2
    uint4 x_unused[4][MT];
    if (group_begin < group_end) load_stage(group_begin / 2, 0);
    for (int gi = group_begin; gi < group_end; gi += 2) {
      const int chunk = gi / 2;
      const int buf = (chunk - group_begin / 2) & 1;
      if (gi + 2 < group_end) {
        load_stage(chunk + 1, buf ^ 1);
        cp_async_wait<1>();  // all but the next A chunk: W groups gi, gi+1 and this A chunk are in
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const int j = gi - group_begin;
      // a W group is asked for as soon as the stage it goes to has been read
      if (gi + 2 < group_end) issue_w(gi + 2, (j + 2) % STAGES);
      cp_async_commit();
      compute(x_unused, gi, j % STAGES, stage[buf]);
      if (gi + 3 < group_end) issue_w(gi + 3, j % STAGES);
      cp_async_commit();
      if (gi + 1 < group_end) compute(x_unused, gi + 1, (j + 1) % STAGES, stage[buf]);
      __syncthreads();
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- split-K: add the partial tiles of the cluster through distributed shared memory
  auto store = [&](int r, float v) {
    const int s = r / (MT * 4), mt = (r / 4) % MT, e = r & 3;
    const int n = n_warp + 16 * s + g + 8 * (e >> 1);
    const int m = 8 * mt + 2 * c + (e & 1);
    if (n < a.N && m < a.M) {
      if (a.bias) v += __bfloat162float(a.bias[n]);
      if (a.residual) v += to_f32(reinterpret_cast<const TOut*>(a.residual)[(size_t)m * a.ldr + n]);
      reinterpret_cast<TOut*>(a.C)[(size_t)m * a.ldc + n] = from_f32<TOut>(v);
    }
  };
  // strip 0 of the warp holds gate rows, strip 1 the up rows of the same 16 outputs
  auto store_swiglu = [&](int r, float gate, float up) {
    const int mt = (r / 4) % MT, e = r & 3;
    const int n = n_warp + g + 8 * (e >> 1);  // gate row; its up row is n + 16
    const int m = 8 * mt + 2 * c + (e & 1);
    if (n + 16 < a.N && m < a.M) {
      const int j = (n_warp >> 1) + g + 8 * (e >> 1);
      reinterpret_cast<TOut*>(a.C)[(size_t)m * a.ldc + j] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
    }
  };
  const bool swiglu = a.epilogue == EPI_SWIGLU;
  if (splits > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    float* red = reinterpret_cast<float*>(smem);  // [R][THREADS]
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[((s * MT + mt) * 4 + r) * THREADS + tid] = acc[s][mt][r];
    cluster.sync();
    const int rank = (int)cluster.block_rank();
    auto total_of = [&](int r) {
      float total = 0.f;
      for (int sp = 0; sp < splits; ++sp) total += cluster.map_shared_rank(red, sp)[r * THREADS + tid];
      return total;
    };
    if (swiglu) {
      for (int r = rank; r < MT * 4; r += splits) store_swiglu(r, total_of(r), total_of(r + MT * 4));
    } else {
      for (int r = rank; r < R; r += splits) store(r, total_of(r));
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
  } else if (swiglu) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int r = 0; r < 4; ++r) store_swiglu(mt * 4 + r, acc[0][mt][r], acc[1][mt][r]);
  } else {
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 4; ++r) store((s * MT + mt) * 4 + r, acc[s][mt][r]);
  }
}

template <int MT, int WARPS, bool STAGED, int PRO, typename TOut>
int launch(const Args& a, int splits, cudaStream_t stream) {
  constexpr int THREADS = WARPS * 32;
  const size_t ring_bytes = (size_t)WARPS * (STAGED ? 3 : 6) * 8192;
  const size_t stage_bytes = STAGED ? 2 * (size_t)(MT * 8) * A_STRIDE : 0;
  const size_t red_bytes = splits > 1 ? (size_t)(2 * MT * 4) * THREADS * sizeof(float) : 0;
  const size_t main_bytes = ring_bytes + stage_bytes;
  const size_t smem = main_bytes > red_bytes ? main_bytes : red_bytes;
  auto kernel = gemm_skinny_kernel<MT, WARPS, STAGED, PRO, TOut>;
  static size_t configured = 0;  // per instantiation; not repeated under graph capture
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + WARPS * 32 - 1) / (WARPS * 32), splits, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
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
  DSP_CUDA(cudaLaunchKernelEx(&cfg, kernel, a));
  return 0;
}

template <int PRO, typename TOut>
int dispatch(const Args& a, int splits, bool narrow, cudaStream_t stream) {
  const int M = a.M;
  if (M <= 8)
    return narrow ? launch<1, 2, false, PRO, TOut>(a, splits, stream) : launch<1, 4, false, PRO, TOut>(a, splits, stream);
  if (M <= 16)
    return narrow ? launch<2, 2, false, PRO, TOut>(a, splits, stream) : launch<2, 4, false, PRO, TOut>(a, splits, stream);
  if (PRO != PRO_NONE) {
    dsp_set_error("dsp_gemm_skinny: a fused prologue takes at most 16 rows, got %d", M);
    return 2;
  }
  if (M <= 32)
    return narrow ? launch<4, 2, true, PRO_NONE, TOut>(a, splits, stream) : launch<4, 4, true, PRO_NONE, TOut>(a, splits, stream);
  return narrow ? launch<8, 2, true, PRO_NONE, TOut>(a, splits, stream) : launch<8, 4, true, PRO_NONE, TOut>(a, splits, stream);
}
}  // namespace

// prologue: 0 none; 1 RMSNorm of A's rows with `gain` and `eps` (M <= 16).
// epilogue: 0 plain; 1 SwiGLU over W rows interleaved in blocks of 16 (C is [M, N/2], no bias or
// residual).  target_ctas: resident CTA slots the launch may fill by splitting K (at most 8 ways).
extern "C" int dsp_gemm_skinny(const void* A, long lda, const void* W, const void* bias,
                               const void* residual, long ldr, void* C, long ldc, int M, int N,
                               int K, int out_dtype, int target_ctas, int prologue,
                               const void* gain, float eps, int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DSP_REQUIRE(M <= 64, "dsp_gemm_skinny: M=%d above 64 rows", M);
  DSP_REQUIRE(K > 0 && K % 8 == 0, "dsp_gemm_skinny: K=%d must be a positive multiple of 8", K);
  DSP_REQUIRE(lda % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0,
              "dsp_gemm_skinny: operands must be 16-byte aligned with a row stride multiple of 8");
  DSP_REQUIRE(prologue != PRO_RMSNORM || (gain != nullptr && ((uintptr_t)gain % 16) == 0),
              "dsp_gemm_skinny: the RMSNorm prologue needs a 16-byte aligned gain");
  Args a;
  a.A = (const bf16*)A;
  a.lda = lda;
  a.W = (const bf16*)W;
  a.bias = (const bf16*)bias;
  a.residual = residual;
  a.ldr = ldr;
  a.C = C;
  a.ldc = ldc;
  a.M = M;
  a.N = N;
  a.K = K;
  a.gain = (const bf16*)gain;
  a.eps = eps;
  a.epilogue = epilogue;
  DSP_REQUIRE(epilogue == EPI_PLAIN || (N % 32 == 0 && bias == nullptr && residual == nullptr),
              "dsp_gemm_skinny: the SwiGLU epilogue needs N in whole blocks of 32 and no bias or residual");
  // CTAs of 64 rows of W, two resident per SM; the K range is split (cluster of up to 8) only as
  // far as the CTAs still fit the resident slots at once.  A negative target selects 128-row CTAs.
  const int groups = (K + 127) / 128;
  const int pairs = (groups + 1) / 2;  // a split covers whole 256-wide chunks
  const int max_splits = pairs < MAX_SPLITS ? pairs : MAX_SPLITS;
  const bool narrow = target_ctas >= 0;
  if (target_ctas < 0) target_ctas = -target_ctas;
  const int n_blocks = narrow ? (N + 63) / 64 : (N + 127) / 128;
  int splits = target_ctas / n_blocks;
  if (splits < 1) splits = 1;
  if (splits > max_splits) splits = max_splits;
  int pairs_per_split = (pairs + splits - 1) / splits;
  splits = (pairs + pairs_per_split - 1) / pairs_per_split;
  a.groups_per_split = pairs_per_split * 2;
  int rc;
  if (out_dtype == DSP_BF16) {
    rc = prologue == PRO_RMSNORM ? dispatch<PRO_RMSNORM, bf16>(a, splits, narrow, stream)
                                 : dispatch<PRO_NONE, bf16>(a, splits, narrow, stream);
  } else if (out_dtype == DSP_F32) {
    rc = prologue == PRO_RMSNORM ? dispatch<PRO_RMSNORM, float>(a, splits, narrow, stream)
                                 : dispatch<PRO_NONE, float>(a, splits, narrow, stream);
  } else {
    DSP_REQUIRE(false, "dsp_gemm_skinny: unknown output dtype %d", out_dtype);
  }
  return rc;
}
