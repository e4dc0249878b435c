// Counter-based normal fill: value = f(seed, tensor ordinal, element index), nothing else.
//
// Element i of tensor `ordinal` comes from Philox-4x32-10 with counter (i / 4 low word, i / 4 high
// word, ordinal, 0) and key (seed low word, seed high word).  The four output words make two
// Box-Muller pairs: words (0, 1) give elements 4b and 4b + 1 (radius * cos, radius * sin), words
// (2, 3) elements 4b + 2 and 4b + 3.  The uniforms are odd multiples of 2^-24 built from the top
// 23 bits of a word, so they are exact in float32 and never 0 or 1.
//
// The logarithm, sine and cosine are written out here in float32 with single, correctly rounded
// operations only (__fadd_rn, __fmul_rn, __fdiv_rn, __fsqrt_rn: never contracted into a fused
// multiply-add), so that the same sequence of operations in any IEEE-754 float32 arithmetic
// (numpy on a CPU) gives the same bits.  out[i] = mean + std * z_i in float32, then rounded once to
// the storage type (optionally through bfloat16 into a float32 buffer, which is what loading a
// bfloat16 checkpoint into the 32-bit engine gives).
#include "common.cuh"

namespace {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0;
  c[1] = n1;
  c[2] = n2;
  c[3] = n3;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// ln(u) for u = odd * 2^-24 in (0, 1): u = m * 2^e with m in [sqrt(1/2), sqrt(2)), ln m by the
// atanh series in s = (m - 1) / (m + 1) up to s^9.
__device__ __forceinline__ float det_log(float u) {
  const uint32_t bits = __float_as_uint(u);
  int e = (int)(bits >> 23) - 127;
  float m = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
  if (m > 1.41421354f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  const float f = __fsub_rn(m, 1.0f);
  const float s = __fdiv_rn(f, __fadd_rn(f, 2.0f));
  const float z = __fmul_rn(s, s);
  float p = __fadd_rn(__fmul_rn(z, 0.222222224f), 0.285714298f);  // 2/9, 2/7
  p = __fadd_rn(__fmul_rn(z, p), 0.400000006f);                   // 2/5
  p = __fadd_rn(__fmul_rn(z, p), 0.666666687f);                   // 2/3
  p = __fadd_rn(__fmul_rn(z, p), 2.0f);
  return __fadd_rn(__fmul_rn((float)e, 0.693147182f), __fmul_rn(s, p));
}

// sin and cos of 2 pi n / 2^24 for an odd n below 2^24: the top three bits of n name the octant,
// the lower 21 the place inside it; the polynomials run on an angle in [0, pi/4].
__device__ __forceinline__ void det_sincos(uint32_t n, float& sn, float& cs) {
  const uint32_t octant = n >> 21;
  uint32_t r = n & 0x1fffffu;
  if (octant & 1u) r = 0x200000u - r;
  const float a = __fmul_rn(__fmul_rn((float)r, 4.76837158e-07f), 0.785398185f);  // r / 2^21 * pi/4
  const float a2 = __fmul_rn(a, a);
  float ps = __fadd_rn(__fmul_rn(a2, 2.75573188e-06f), -1.98412701e-04f);  // 1/9!, -1/7!
  ps = __fadd_rn(__fmul_rn(a2, ps), 8.33333377e-03f);                      // 1/5!
  ps = __fadd_rn(__fmul_rn(a2, ps), -0.166666672f);                        // -1/3!
  ps = __fadd_rn(__fmul_rn(a2, ps), 1.0f);
  const float s = __fmul_rn(a, ps);
  float pc = __fadd_rn(__fmul_rn(a2, -2.75573188e-07f), 2.48015876e-05f);  // -1/10!, 1/8!
  pc = __fadd_rn(__fmul_rn(a2, pc), -1.38888892e-03f);                     // -1/6!
  pc = __fadd_rn(__fmul_rn(a2, pc), 4.16666679e-02f);                      // 1/4!
  pc = __fadd_rn(__fmul_rn(a2, pc), -0.5f);
  const float c = __fadd_rn(__fmul_rn(a2, pc), 1.0f);
  // octants 0..7 of the full turn: which of (s, c) is the sine, and the signs
  const bool swap = ((octant + 1u) >> 1) & 1u;  // octants 1, 2, 5, 6
  const float sv = swap ? c : s, cv = swap ? s : c;
  sn = (octant >= 4u) ? -sv : sv;
  cs = (octant >= 2u && octant <= 5u) ? -cv : cv;
}

__device__ __forceinline__ void normal_pair(uint32_t w0, uint32_t w1, float& z0, float& z1) {
  const float u = __fmul_rn((float)(2u * (w0 >> 9) + 1u), 5.96046448e-08f);  // odd * 2^-24
  const float radius = __fsqrt_rn(__fmul_rn(-2.0f, det_log(u)));
  float sn, cs;
  det_sincos(2u * (w1 >> 9) + 1u, sn, cs);
  z0 = __fmul_rn(radius, cs);
  z1 = __fmul_rn(radius, sn);
}

template <typename T>
__global__ void fill_normal_kernel(T* out, long n, uint32_t seed_lo, uint32_t seed_hi, uint32_t ordinal,
                                   float mean, float std, int through_bf16) {
  const long blocks = (n + 3) / 4;
  for (long b = (long)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += (long)gridDim.x * blockDim.x) {
    uint32_t c[4] = {(uint32_t)((unsigned long)b & 0xffffffffu), (uint32_t)((unsigned long)b >> 32), ordinal, 0u};
    philox4x32_10(c, seed_lo, seed_hi);
    float z[4];
    normal_pair(c[0], c[1], z[0], z[1]);
    normal_pair(c[2], c[3], z[2], z[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long i = 4 * b + j;
      if (i < n) {
        float v = __fadd_rn(mean, __fmul_rn(std, z[j]));
        if (through_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        out[i] = from_f32<T>(v);
      }
    }
  }
}
}  // namespace

// out: n elements of float32 (dtype 0) or bfloat16 (dtype 1), contiguous.  through_bf16: round to
// bfloat16 first even when the buffer is float32.
extern "C" int dsp_fill_normal(void* out, long n, unsigned long long seed, unsigned int ordinal, float mean,
                               float std, int dtype, int through_bf16, cudaStream_t stream) {
  if (n <= 0) return 0;
  DSP_REQUIRE(dtype == DSP_F32 || dtype == DSP_BF16, "dsp_fill_normal: unknown dtype %d", dtype);
  const long blocks = (n + 3) / 4;
  const int sms = dsp_num_sms() > 0 ? dsp_num_sms() : 1;
  const long want = (blocks + 255) / 256;
  const int grid = (int)(want < (long)sms * 32 ? want : (long)sms * 32);
  const uint32_t lo = (uint32_t)(seed & 0xffffffffull), hi = (uint32_t)(seed >> 32);
  if (dtype == DSP_F32)
    fill_normal_kernel<float><<<grid, 256, 0, stream>>>((float*)out, n, lo, hi, ordinal, mean, std, through_bf16);
  else
    fill_normal_kernel<bf16><<<grid, 256, 0, stream>>>((bf16*)out, n, lo, hi, ordinal, mean, std, through_bf16);
  DSP_CHECK_LAUNCH("dsp_fill_normal");
  return 0;
}
