// Causal grouped-query attention over the paged key/value cache, all arithmetic in 32-bit.
//
// One block per (query token, KV head); the G = H / KVH query heads of the group share every
// key and value load.  The query at absolute position p sees keys b with
//     max(0, p - window + 1) <= b <= p        (window == 0: every key from 0)
// which is the lower-right aligned causal mask for a portion of a prompt on top of cached
// tokens, and a single decoded token alike.  Online softmax (running max m, running sum l)
// over tiles of 128 keys.  Any head_dim that is a multiple of 4 (float) / 8 (bfloat16) up to
// 512, any G.  This kernel is the attention of the 32-bit path and the fallback of the
// bfloat16 path for head sizes the tensor-core kernel is not built for.
//
// q:   element (t, head, d) at q[t * q_stride + head * D + d]
// out: element (t, head, d) at out[t * out_stride + head * D + d]
// pools: [num_pages, KVH, page_size, D]; page = page_table[seq * pt_stride + b / page_size]
#include "common.cuh"

namespace {
constexpr int THREADS = 128;   // = keys per tile
constexpr int GCHUNK = 8;      // query heads handled per pass
constexpr int DPT = 4;         // output dims per thread: head_dim <= THREADS * DPT

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_generic_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k_pool,
                    const T* __restrict__ v_pool, const int* __restrict__ page_table,
                    int pt_stride, const int* __restrict__ positions,
                    const int* __restrict__ seq_of_token, T* __restrict__ out, long out_stride,
                    int H, int KVH, int D, int page_size, int num_pages, int window, float scale,
                    int* err) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [GCHUNK][D]
  float* ps = qs + GCHUNK * D;            // [GCHUNK][THREADS]
  long* slot = (long*)(ps + GCHUNK * THREADS);  // [THREADS] element offset of each key row
  __shared__ float red[GCHUNK][THREADS / 32];

  const int t = blockIdx.x, kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = positions[t];
  if (pos < 0) return;
  const int seq = seq_of_token[t];
  const int G = H / KVH;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int hi = pos;
  const int* table = page_table + (size_t)seq * pt_stride;

  for (int g0 = 0; g0 < G; g0 += GCHUNK) {
    const int gn = min(GCHUNK, G - g0);
    __syncthreads();
    for (int i = tid; i < gn * D; i += THREADS) {
      const int g = i / D, d = i % D;
      qs[g * D + d] = to_f32(q[(size_t)t * q_stride + (size_t)(kvh * G + g0 + g) * D + d]) * scale;
    }
    float m[GCHUNK], l[GCHUNK], acc[GCHUNK][DPT];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int j = 0; j < DPT; ++j) acc[g][j] = 0.f;
    }
    __syncthreads();

    for (int kt = lo; kt <= hi; kt += THREADS) {
      const int key = kt + tid;
      const bool valid = key <= hi;
      float s[GCHUNK];
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) s[g] = -INFINITY;
      long off = -1;
      if (valid) {
        const int page = table[key / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, DSP_ERR_BAD_PAGE);
        } else {
          off = (((long)page * KVH + kvh) * page_size + (key % page_size)) * D;
          const T* kr = k_pool + off;
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g) s[g] = 0.f;
          for (int d = 0; d < D; ++d) {
            const float kv = to_f32(kr[d]);
#pragma unroll
            for (int g = 0; g < GCHUNK; ++g)
              if (g < gn) s[g] = fmaf(qs[g * D + d], kv, s[g]);
          }
        }
      }
      slot[tid] = off;
      // tile maxima, one per head
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) {
        const float wm = warp_max(s[g]);
        if (lane == 0) red[g][warp] = wm;
      }
      __syncthreads();
      float alpha[GCHUNK], p[GCHUNK];
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) {
        float tm = red[g][0];
#pragma unroll
        for (int w = 1; w < THREADS / 32; ++w) tm = fmaxf(tm, red[g][w]);
        const float m_new = fmaxf(m[g], tm);
        // m_new stays -inf only for heads beyond gn or when every page id was bad
        alpha[g] = (m_new == -INFINITY) ? 1.f : expf(m[g] - m_new);
        p[g] = (off >= 0 && g < gn) ? expf(s[g] - m_new) : 0.f;
        m[g] = m_new;
        ps[g * THREADS + tid] = p[g];
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) {
        const float ws = warp_sum(p[g]);
        if (lane == 0) red[g][warp] = ws;
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) {
        float ts = red[g][0];
#pragma unroll
        for (int w = 1; w < THREADS / 32; ++w) ts += red[g][w];
        l[g] = l[g] * alpha[g] + ts;
#pragma unroll
        for (int j = 0; j < DPT; ++j) acc[g][j] *= alpha[g];
      }
      // weighted sum of values: thread owns dims tid, tid+128, ...
      const int nkeys = min(THREADS, hi - kt + 1);
      for (int j = 0; j < nkeys; ++j) {
        const long vo = slot[j];
        if (vo < 0) continue;
        const T* vr = v_pool + vo;
#pragma unroll
        for (int dd = 0; dd < DPT; ++dd) {
          const int d = tid + dd * THREADS;
          if (d < D) {
            const float vv = to_f32(vr[d]);
#pragma unroll
            for (int g = 0; g < GCHUNK; ++g)
              if (g < gn) acc[g][dd] = fmaf(ps[g * THREADS + j], vv, acc[g][dd]);
          }
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      if (g >= gn) continue;
      const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
#pragma unroll
      for (int dd = 0; dd < DPT; ++dd) {
        const int d = tid + dd * THREADS;
        if (d < D)
          out[(size_t)t * out_stride + (size_t)(kvh * G + g0 + g) * D + d] =
              from_f32<T>(acc[g][dd] * inv);
      }
    }
  }
}
}  // namespace

extern "C" int dsp_attn_generic(const void* q, long q_stride, const void* k_pool,
                                const void* v_pool, const int* page_table, int pt_stride,
                                const int* positions, const int* seq_of_token, void* out,
                                long out_stride, int T, int H, int KVH, int D, int page_size,
                                int num_pages, int window, float scale, int dtype,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(KVH > 0 && H % KVH == 0, "dsp_attn_generic: H=%d is not a multiple of KVH=%d", H, KVH);
  DSP_REQUIRE(D > 0 && D <= THREADS * DPT, "dsp_attn_generic: head_dim=%d outside (0, %d]", D,
              THREADS * DPT);
  DSP_REQUIRE(KVH <= 65535, "dsp_attn_generic: too many KV heads");
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_attn_generic: no device error word");
  const size_t smem = (size_t)(GCHUNK * D + GCHUNK * THREADS) * sizeof(float) + THREADS * sizeof(long);
  dim3 grid(T, KVH);
  if (dtype == DSP_F32) {
    static size_t configured = 0;
    if (smem > configured) {
      DSP_CUDA(cudaFuncSetAttribute(attn_generic_kernel<float>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured = smem;
    }
    attn_generic_kernel<float><<<grid, THREADS, smem, stream>>>(
        (const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, page_table, pt_stride,
        positions, seq_of_token, (float*)out, out_stride, H, KVH, D, page_size, num_pages, window,
        scale, err);
  } else if (dtype == DSP_BF16) {
    static size_t configured = 0;
    if (smem > configured) {
      DSP_CUDA(cudaFuncSetAttribute(attn_generic_kernel<bf16>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured = smem;
    }
    attn_generic_kernel<bf16><<<grid, THREADS, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, page_table, pt_stride,
        positions, seq_of_token, (bf16*)out, out_stride, H, KVH, D, page_size, num_pages, window,
        scale, err);
  } else {
    DSP_REQUIRE(false, "dsp_attn_generic: unknown dtype %d", dtype);
  }
  DSP_CHECK_LAUNCH("dsp_attn_generic");
  return 0;
}
