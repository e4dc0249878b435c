// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ residual[M,N]) on the 32-bit FMA units.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision
// mode) and the catch-all for sizes the tensor-core kernels refuse.  Every output element is
// one FMA chain over k = 0..K-1 in ascending order, so a row's result does not depend on
// which other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ A, long lda, const TIn* __restrict__ W,
                 const TIn* __restrict__ bias, const TOut* __restrict__ residual, long ldr,
                 TOut* __restrict__ C, long ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // outputs rows ty*4.., cols tx*4..
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, c = idx % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32(bias[gn]);
      if (residual) v += to_f32(residual[(size_t)gm * ldr + gn]);
      C[(size_t)gm * ldc + gn] = from_f32<TOut>(v);
    }
  }
}

template <typename TIn, typename TOut>
int launch(const void* A, long lda, const void* W, const void* bias, const void* residual, long ldr,
           void* C, long ldc, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  DSP_REQUIRE(grid.y <= 65535, "dsp_gemm_simt: M=%d too large for one launch", M);
  gemm_simt_kernel<TIn, TOut><<<grid, 256, 0, stream>>>(
      (const TIn*)A, lda, (const TIn*)W, (const TIn*)bias, (const TOut*)residual, ldr, (TOut*)C, ldc,
      M, N, K);
  DSP_CHECK_LAUNCH("dsp_gemm_simt");
  return 0;
}
}  // namespace

// in_dtype: type of A, W and bias.  out_dtype: type of C and residual.
extern "C" int dsp_gemm_simt(const void* A, long lda, const void* W, const void* bias,
                             const void* residual, long ldr, void* C, long ldc, int M, int N, int K,
                             int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DSP_REQUIRE(K > 0, "dsp_gemm_simt: K=%d", K);
  if (in_dtype == DSP_F32 && out_dtype == DSP_F32)
    return launch<float, float>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, stream);
  if (in_dtype == DSP_BF16 && out_dtype == DSP_BF16)
    return launch<bf16, bf16>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, stream);
  if (in_dtype == DSP_BF16 && out_dtype == DSP_F32)
    return launch<bf16, float>(A, lda, W, bias, residual, ldr, C, ldc, M, N, K, stream);
  DSP_REQUIRE(false, "dsp_gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
