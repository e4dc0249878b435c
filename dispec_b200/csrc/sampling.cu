// Token choice from 32-bit logits: argmax (ties to the lowest index) and temperature sampling
// with top-k and top-p masks, one block per row.
//
// Sampling follows puneethgv/DiSpec dispec/sampling.py:26-75: x = logits / T; top-k keeps
// every x >= the k-th largest (ties stay); top-p walks x in descending order and drops a
// token when the probability mass before it exceeds top_p (the first always stays); the
// token is drawn from softmax over what is left.  The draw is the inverse CDF in vocabulary
// order at a uniform number u in [0, 1) that the host supplies per row, so a CPU
// implementation can replay it.  All selections are deterministic: counts are integer
// histograms, top-p mass is accumulated in 2^-40 fixed point, sums run in a fixed order.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ int block_argmax(const float* x, int V, ArgMax* scratch) {
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) best = better(best, ArgMax{x[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  ArgMax total = scratch[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) total = better(total, scratch[w]);
  if (total.i == 0x7fffffff) total.i = 0;  // a row of NaN or -inf: index 0
  return total.i;
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, long stride, int V, int* __restrict__ out) {
  __shared__ ArgMax scratch[32];
  const int r = blockIdx.x;
  const int idx = block_argmax(logits + (size_t)r * stride, V, scratch);
  if (threadIdx.x == 0) out[r] = idx;
}

// Two-stage form for large vocabularies: grid (rows, chunks); each block reduces one chunk of a
// row to (value, index), a second small kernel reduces the chunks in index order.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, long stride, int V, int chunk,
                      float* __restrict__ part_val, int* __restrict__ part_idx) {
  __shared__ ArgMax scratch[32];
  const int r = blockIdx.x, c = blockIdx.y;
  const int begin = c * chunk, end = min(V, begin + chunk);
  const float* x = logits + (size_t)r * stride;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, ArgMax{x[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgMax total = scratch[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) total = better(total, scratch[w]);
    part_val[(size_t)r * gridDim.y + c] = total.v;
    part_idx[(size_t)r * gridDim.y + c] = total.i;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int chunks, int* __restrict__ out) {
  const int r = blockIdx.x;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < chunks; c += 32)
    best = better(best, ArgMax{part_val[(size_t)r * chunks + c], part_idx[(size_t)r * chunks + c]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// inclusive scan over the block in thread order; returns this thread's inclusive value and
// the block total through *total.  scratch: 32 entries.
template <typename V>
__device__ __forceinline__ V block_scan(V v, V* scratch, V* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const V n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = v;
  __syncthreads();
  V before = 0, sum = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    if (w < warp) before += scratch[w];
    sum += scratch[w];
  }
  *total = sum;
  return v + before;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  __shared__ ArgMax am_scratch[32];
  __shared__ float f_scratch[32];
  __shared__ int i_scratch[32];
  __shared__ int cnt_hist[256];
  __shared__ unsigned long long mass_hist[256];
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_k;
  __shared__ unsigned long long sh_above;
  __shared__ int sh_ties, sh_found;
  __shared__ unsigned long long sh_tie_mass;

  const int r = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)r * stride;
  const float T = temperature[r];
  if (!(T > 0.f)) {
    const int idx = block_argmax(x, V, am_scratch);
    if (tid == 0) out[r] = idx;
    return;
  }

  // ---- top-k: key of the k-th largest x/T (0 keeps everything)
  uint32_t kth_key = 0;
  int k = top_k[r];
  if (k > 0 && k < V) {
    uint32_t prefix = 0, mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += THREADS) cnt_hist[b] = 0;
      __syncthreads();
      for (int i = tid; i < V; i += THREADS) {
        const uint32_t key = order_key(x[i] / T);
        if ((key & mask) == prefix) atomicAdd(&cnt_hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, b = 255;
        for (; b > 0; --b) {
          if (cum + cnt_hist[b] >= k) break;
          cum += cnt_hist[b];
        }
        sh_k = k - cum;
        sh_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
      k = sh_k;
      prefix = sh_prefix;
      mask |= 255u << shift;
      __syncthreads();
    }
    kth_key = prefix;
  }

  // ---- max and normaliser over what top-k left
  float mx = -INFINITY;
  for (int i = tid; i < V; i += THREADS) {
    const float v = x[i] / T;
    if (order_key(v) >= kth_key) mx = fmaxf(mx, v);
  }
  mx = block_max(mx, f_scratch);
  float zsum = 0.f;
  for (int i0 = 0; i0 < V; i0 += THREADS) {  // chunk order is fixed: deterministic
    const int i = i0 + tid;
    if (i < V) {
      const float v = x[i] / T;
      if (order_key(v) >= kth_key) zsum += expf(v - mx);
    }
  }
  const float Z = block_sum(zsum, f_scratch);

  // ---- top-p: smallest kept value v* and how many of its ties stay
  uint32_t vstar_key = 0;
  int keep_ties = 0x7fffffff;
  const float p = top_p[r];
  if (p < 1.f) {
    const float to_fixed = 1099511627776.f / Z;  // 2^40 / Z
    const unsigned long long thresh = (unsigned long long)((double)fmaxf(p, 0.f) * 1099511627776.0);
    uint32_t prefix = 0, mask = 0;
    unsigned long long above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += THREADS) {
        cnt_hist[b] = 0;
        mass_hist[b] = 0ull;
      }
      __syncthreads();
      for (int i = tid; i < V; i += THREADS) {
        const float v = x[i] / T;
        const uint32_t key = order_key(v);
        if (key >= kth_key && (key & mask) == prefix) {
          const int b = (key >> shift) & 255u;
          atomicAdd(&cnt_hist[b], 1);
          atomicAdd(&mass_hist[b], __float2ull_rd(expf(v - mx) * to_fixed));
        }
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long run = above, best_above = above;
        int best = -1;
        for (int b = 255; b >= 0; --b) {
          if (cnt_hist[b] == 0) continue;
          if (run <= thresh || best < 0) {
            best = b;
            best_above = run;
          } else {
            break;
          }
          run += mass_hist[b];
        }
        if (best < 0) best = 0;
        sh_prefix = prefix | ((uint32_t)best << shift);
        sh_above = best_above;
        sh_ties = cnt_hist[best];
        sh_tie_mass = mass_hist[best];
      }
      __syncthreads();
      prefix = sh_prefix;
      above = sh_above;
      mask |= 255u << shift;
      __syncthreads();
    }
    vstar_key = prefix;
    const int ties = sh_ties;
    const unsigned long long each = ties > 0 ? sh_tie_mass / (unsigned long long)ties : 0ull;
    if (each > 0ull && thresh >= above) {
      const unsigned long long extra = (thresh - above) / each;
      keep_ties = (int)min((unsigned long long)ties, extra + 1ull);
    } else {
      keep_ties = each > 0ull ? 1 : ties;
    }
  }

  // ---- two ordered passes: mass of the kept set, then the inverse CDF at u
  float kept_total = 0.f;
  for (int pass = 0; pass < 2; ++pass) {
    const float target = uniform[r] * kept_total;
    float run = 0.f;
    int ties_seen = 0;
    int last_kept = -1;
    if (tid == 0) sh_found = 0x7fffffff;
    __syncthreads();
    for (int i0 = 0; i0 < V; i0 += THREADS) {
      const int i = i0 + tid;
      float w = 0.f;
      int tie = 0;
      uint32_t key = 0;
      if (i < V) {
        const float v = x[i] / T;
        key = order_key(v);
        if (key >= kth_key && key >= vstar_key) {
          w = expf(v - mx);
          tie = (key == vstar_key && keep_ties != 0x7fffffff) ? 1 : 0;
        }
      }
      int tie_total = 0;
      int tie_incl = tie;
      if (keep_ties != 0x7fffffff) tie_incl = block_scan<int>(tie, i_scratch, &tie_total);
      if (tie && ties_seen + tie_incl > keep_ties) w = 0.f;
      ties_seen += tie_total;
      float w_total;
      const float incl = block_scan<float>(w, f_scratch, &w_total);
      if (w > 0.f) last_kept = i;
      if (pass == 1) {
        if (w > 0.f && run + incl > target) atomicMin(&sh_found, i);
        __syncthreads();
        if (sh_found != 0x7fffffff) break;
      }
      run += w_total;
    }
    if (pass == 0) {
      kept_total = run;
      __syncthreads();
    } else {
      // rounding may leave the target just above the last partial sum: take the last kept token
      int lk = last_kept;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
      __syncthreads();
      if ((tid & 31) == 0) i_scratch[tid >> 5] = lk;
      __syncthreads();
      if (tid == 0) {
        int found = sh_found;
        if (found == 0x7fffffff) {
          int m = -1;
          for (int w2 = 0; w2 < THREADS / 32; ++w2) m = max(m, i_scratch[w2]);
          found = m < 0 ? 0 : m;
        }
        out[r] = found;
      }
    }
  }
}
}  // namespace

// chunks > 1 with scratch for n * chunks (value, index) pairs selects the two-stage form.
extern "C" int dsp_argmax(const float* logits, long stride, int n, int V, int* out, int chunks,
                          float* part_val, int* part_idx, cudaStream_t stream) {
  if (n == 0) return 0;
  DSP_REQUIRE(V > 0, "dsp_argmax: V=%d", V);
  if (chunks > 1 && part_val != nullptr && part_idx != nullptr) {
    DSP_REQUIRE(chunks <= 65535, "dsp_argmax: too many chunks");
    const int chunk = (V + chunks - 1) / chunks;
    argmax_partial_kernel<<<dim3(n, chunks), 256, 0, stream>>>(logits, stride, V, chunk, part_val, part_idx);
    argmax_final_kernel<<<n, 32, 0, stream>>>(part_val, part_idx, chunks, out);
  } else {
    argmax_kernel<<<n, THREADS, 0, stream>>>(logits, stride, V, out);
  }
  DSP_CHECK_LAUNCH("dsp_argmax");
  return 0;
}

// temperature[r] <= 0 selects argmax for that row; top_k[r] == 0 and top_p[r] >= 1 switch the
// masks off; uniform[r] in [0, 1).
extern "C" int dsp_sample(const float* logits, long stride, int n, int V, const float* temperature,
                          const int* top_k, const float* top_p, const float* uniform, int* out,
                          cudaStream_t stream) {
  if (n == 0) return 0;
  DSP_REQUIRE(V > 0, "dsp_sample: V=%d", V);
  sample_kernel<<<n, THREADS, 0, stream>>>(logits, stride, V, temperature, top_k, top_p, uniform,
                                           out);
  DSP_CHECK_LAUNCH("dsp_sample");
  return 0;
}

// ------------------------------------------------------------------ argmax without allocation
// The two-stage argmax with its scratch inside the library image; see no_alloc.h for who needs
// it and for the rules (size limit, first call, sharing).
#include "no_alloc.h"

namespace {
constexpr int STATIC_MAX_ROWS = 1024;
constexpr int STATIC_MAX_CHUNKS = 64;
}  // namespace

// [STATIC_MAX_ROWS * STATIC_MAX_CHUNKS] floats, then as many ints.  In host code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char
    g_argmax_static_scratch[STATIC_MAX_ROWS * STATIC_MAX_CHUNKS * (sizeof(float) + sizeof(int))];

extern "C" int dsp_argmax_static_max_rows(void) { return STATIC_MAX_ROWS; }

extern "C" int dsp_argmax_static(const float* logits, long stride, int n, int V, int* out,
                                 cudaStream_t stream) {
  if (n == 0) return 0;
  DSP_REQUIRE(n > 0 && n <= STATIC_MAX_ROWS,
              "dsp_argmax_static: %d rows, the built-in scratch holds at most %d", n, STATIC_MAX_ROWS);
  DSP_REQUIRE(V > 0, "dsp_argmax_static: V=%d", V);
  DSP_REQUIRE(logits != nullptr && out != nullptr, "dsp_argmax_static: null pointer");
  // set-up, once per device, with that device current
  static unsigned char* address[64] = {nullptr};
  int dev = 0;
  DSP_CUDA(cudaGetDevice(&dev));
  DSP_REQUIRE(dev >= 0 && dev < 64, "dsp_argmax_static: device index %d out of range", dev);
  if (address[dev] == nullptr) {
    unsigned char* p = nullptr;
    DSP_CUDA(cudaGetSymbolAddress((void**)&p, g_argmax_static_scratch));
    DSP_REQUIRE(p != nullptr, "dsp_argmax_static: the scratch array has no device address");
    address[dev] = p;
  }
  float* part_val = reinterpret_cast<float*>(address[dev]);
  int* part_idx = reinterpret_cast<int*>(address[dev] + (size_t)STATIC_MAX_ROWS * STATIC_MAX_CHUNKS * sizeof(float));
  int chunks = (V + 4095) / 4096;
  if (chunks > STATIC_MAX_CHUNKS) chunks = STATIC_MAX_CHUNKS;
  const int chunk = (V + chunks - 1) / chunks;
  argmax_partial_kernel<<<dim3(n, chunks), 256, 0, stream>>>(logits, stride, V, chunk, part_val, part_idx);
  argmax_final_kernel<<<n, 32, 0, stream>>>(part_val, part_idx, chunks, out);
  DSP_CHECK_LAUNCH("dsp_argmax_static");
  return 0;
}
