// Merges the partial results of split attention: for each (token, head) row the splits hold an
// unnormalised output o_s, a running maximum m_s (base-2 exponent domain) and a sum l_s.
//   M = max_s m_s;  w_s = 2^(m_s - M);  out = sum_s w_s o_s / sum_s w_s l_s
// A split that saw no key has l_s = 0 and m_s = -inf and contributes nothing.
#include "common.cuh"

// One block per row, at most 32 splits.  Every warp reads the row's (m_s, l_s), one split per
// lane, and finds M, the weights and the sum by shuffles (no loop of dependent loads); each thread
// then requests the splits' outputs of its element eight at a time before it adds them in split
// order.
constexpr int COMBINE_MAX_SPLITS = 32;

template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    T* __restrict__ out, long out_stride, int H, int D, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;  // t * H + h
  const size_t t = row / H;
  const int h = (int)(row % H);
  const int lane = threadIdx.x & 31;
  float m = -INFINITY, l = 0.f;
  if (lane < splits) {
    const float2 ml = reinterpret_cast<const float2*>(part_ml)[row * splits + lane];
    m = ml.x;
    l = ml.y;
  }
  const float M = warp_max(m);
  const float w = m == -INFINITY ? 0.f : exp2f(m - M);
  const float L = warp_sum(w * l);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  const float* po = part_o + row * splits * D;
  for (int d0 = (int)threadIdx.x - lane; d0 < D; d0 += blockDim.x) {  // the same trips for a whole warp (shuffles)
    const int d = d0 + lane;
    const bool on = d < D;
    float acc = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float ws = __shfl_sync(0xffffffffu, w, (s0 + j) & 31);
        // a split that saw no key has weight 0 and an output that was never written: not read
        v[j] = (on && s0 + j < splits && ws != 0.f) ? ws * po[(size_t)(s0 + j) * D + d] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += v[j];
    }
    if (on) out[t * out_stride + (size_t)h * D + d] = from_f32<T>(acc * inv);
  }
}

extern "C" int dsp_attn_combine(const float* part_o, const float* part_ml, void* out, long out_stride,
                                int num_tokens, int H, int D, int splits, int dtype,
                                cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  DSP_REQUIRE(splits >= 1 && splits <= COMBINE_MAX_SPLITS, "dsp_attn_combine: splits=%d outside 1..%d", splits,
              COMBINE_MAX_SPLITS);
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
