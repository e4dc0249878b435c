// Merges the partial results of split attention: for each (token, head) row the splits hold an
// unnormalised output o_s, a running maximum m_s (base-2 exponent domain) and a sum l_s.
//   M = max_s m_s;  w_s = 2^(m_s - M);  out = sum_s w_s o_s / sum_s w_s l_s
// A split that saw no key has l_s = 0 and m_s = -inf and contributes nothing.
#include "common.cuh"

template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    T* __restrict__ out, long out_stride, int H, int D, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;  // t * H + h
  const size_t t = row / H;
  const int h = (int)(row % H);
  const float* ml = part_ml + row * splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = ml[2 * s];
    if (m != -INFINITY) L += exp2f(m - M) * ml[2 * s + 1];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = ml[2 * s];
      if (m != -INFINITY) acc += exp2f(m - M) * part_o[(row * splits + s) * D + d];
    }
    out[t * out_stride + (size_t)h * D + d] = from_f32<T>(acc * inv);
  }
}

extern "C" int dsp_attn_combine(const float* part_o, const float* part_ml, void* out, long out_stride,
                                int num_tokens, int H, int D, int splits, int dtype,
                                cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  DSP_REQUIRE(splits >= 1, "dsp_attn_combine: splits=%d", splits);
  const int rows = num_tokens * H;
  const int threads = D >= 128 ? 128 : 64;
  if (dtype == DSP_BF16)
    DSP_CUDA(launch_pdl(attn_combine_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, part_o, part_ml, (bf16*)out, out_stride, H, D, splits));
  else if (dtype == DSP_F32)
    DSP_CUDA(launch_pdl(attn_combine_kernel<float>, dim3(rows), dim3(threads), 0, stream, part_o, part_ml, (float*)out, out_stride, H, D, splits));
  else
    DSP_REQUIRE(false, "dsp_attn_combine: unknown dtype %d", dtype);
  DSP_CHECK_LAUNCH("dsp_attn_combine");
  return 0;
}
