// Memory-bound kernels of the step: embedding gather, RMSNorm (with and without the fused
// residual sum), SwiGLU, and rotary position encoding fused with the paged key/value write.
// All arithmetic is 32-bit; storage is float or bfloat16 (template parameter).
#include "common.cuh"

// ---------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :].  An id outside [0, vocab) writes zeros and sets the error word.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             T* __restrict__ out, int hidden, int vocab, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  T* dst = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>(0.f);
    return;
  }
  const T* src = table + (size_t)id * hidden;
  const int vec = 16 / sizeof(T);
  if ((hidden % vec) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < hidden / vec; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

extern "C" int dsp_embed(const void* table, const int* ids, void* out, int T, int hidden,
                         int vocab, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_embed: no device error word");
  if (dtype == DSP_F32)
    DSP_CUDA(launch_pdl(embed_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)table, ids, (float*)out, hidden, vocab, err));
  else if (dtype == DSP_BF16)
    DSP_CUDA(launch_pdl(embed_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)table, ids, (bf16*)out, hidden, vocab, err));
  else
    DSP_REQUIRE(false, "dsp_embed: unknown dtype %d", dtype);
  DSP_CHECK_LAUNCH("dsp_embed");
  return 0;
}

// ------------------------------------------------------------------ tokens fed on the device
// ids[t] = prev[src[t]] where src[t] >= 0: the token a request sampled in the previous step becomes
// its input in this one without a round trip through the host.  A source row outside prev is
// recorded in the device error word; the value itself is range-checked by the embedding kernel.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ src,
                                   const int* __restrict__ prev, int n, int n_prev, int* err) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int s = src[t];
  if (s < 0) return;
  if (s >= n_prev) {
    atomicOr(err, DSP_ERR_BAD_TOKEN);
    return;
  }
  ids[t] = prev[s];
}

extern "C" int dsp_feed_tokens(int* ids, const int* src, const int* prev, int n, int n_prev,
                               cudaStream_t stream) {
  if (n == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_feed_tokens: no device error word");
  DSP_REQUIRE(ids && src && prev && n_prev > 0, "dsp_feed_tokens: missing operand");
  feed_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, src, prev, n, n_prev, err);
  DSP_CHECK_LAUNCH("dsp_feed_tokens");
  return 0;
}

// ------------------------------------------------------------------------------ RMSNorm
// y = w * round_T( x * rsqrt(mean(x^2) + eps) ), x read as 32-bit, the product with w
// rounded once more to T (for float both roundings are the identity).
// With `delta`: s = x + delta in 32-bit, rounded to T; the norm is taken of the rounded sum
// and, if `write_back`, the sum replaces x.  `rows` (optional) gathers input rows; output
// row i is dense.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta,
                               const T* __restrict__ w, T* __restrict__ y,
                               const int* __restrict__ rows, int hidden, float eps,
                               int write_back) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t in_row = rows ? (size_t)rows[r] : (size_t)r;
  T* xr = x + in_row * hidden;
  const T* dr = delta ? delta + in_row * hidden : nullptr;
  T* yr = y + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32(xr[i]);
    if (dr) {
      v = to_f32(from_f32<T>(v + to_f32(dr[i])));
      // stash the rounded sum in y so that the second pass need not redo the sum
      yr[i] = from_f32<T>(v);
      if (write_back) xr[i] = from_f32<T>(v);
    }
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = dr ? to_f32(yr[i]) : to_f32(xr[i]);
    const T n = from_f32<T>(v * rstd);
    yr[i] = from_f32<T>(to_f32(w[i]) * to_f32(n));
  }
}

// Fast form of the same computation for rows whose bytes are a multiple of 16 and that fit in
// registers (hidden <= 256 threads * 4 vectors): one read of x (and delta), one write of y.
// (A warp per row with all of a lane's loads in flight, for the 2,048 rows of a prompt's portion,
// was measured and dropped: alone as fast, the prefill step 2 % slower at a width of 1,536 and
// 10 % at 3,584, where it needs 224 registers.)
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T, int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ w,
                   T* __restrict__ y, const int* __restrict__ rows, int hidden, float eps,
                   int write_back) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t in_row = rows ? (size_t)rows[r] : (size_t)r;
  const int nvec = hidden / N;
  uint4* xr = reinterpret_cast<uint4*>(x + in_row * hidden);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + in_row * hidden) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)r * hidden);
  float vals[VPT][N];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      uint4 raw = xr[i];
      const T* e = reinterpret_cast<const T*>(&raw);
      if (dr) {
        uint4 draw = dr[i];
        const T* d = reinterpret_cast<const T*>(&draw);
        uint4 sum_raw;
        T* sp = reinterpret_cast<T*>(&sum_raw);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          sp[k] = from_f32<T>(to_f32(e[k]) + to_f32(d[k]));
          vals[j][k] = to_f32(sp[k]);
        }
        if (write_back) xr[i] = sum_raw;
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k) vals[j][k] = to_f32(e[k]);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) ss += vals[j][k] * vals[j][k];
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      uint4 wraw = wr[i];
      const T* wv = reinterpret_cast<const T*>(&wraw);
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const T n = from_f32<T>(vals[j][k] * rstd);
        o[k] = from_f32<T>(to_f32(wv[k]) * to_f32(n));
      }
      yr[i] = out;
    }
  }
}

template <typename T>
static bool launch_rmsnorm_vec(void* x, const void* delta, const void* w, void* y, const int* rows,
                               int n_rows, int hidden, float eps, int write_back,
                               cudaStream_t stream) {
  constexpr int N = Vec16<T>::N;
  if (hidden % N != 0) return false;
  const uintptr_t bits = (uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)y;
  if (bits % 16 != 0) return false;
  const int nvec = hidden / N;
  if (nvec <= 256)
    launch_pdl(rmsnorm_vec_kernel<T, 1>, dim3(n_rows), dim3(256), 0, stream, (T*)x, (const T*)delta, (const T*)w, (T*)y, rows, hidden, eps, write_back);
  else if (nvec <= 512)
    launch_pdl(rmsnorm_vec_kernel<T, 2>, dim3(n_rows), dim3(256), 0, stream, (T*)x, (const T*)delta, (const T*)w, (T*)y, rows, hidden, eps, write_back);
  else if (nvec <= 1024)
    launch_pdl(rmsnorm_vec_kernel<T, 4>, dim3(n_rows), dim3(256), 0, stream, (T*)x, (const T*)delta, (const T*)w, (T*)y, rows, hidden, eps, write_back);
  else
    return false;
  return true;
}

extern "C" int dsp_rmsnorm(void* x, const void* delta, const void* w, void* y, const int* rows,
                           int n_rows, int hidden, float eps, int write_back, int dtype,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DSP_REQUIRE(hidden > 0, "dsp_rmsnorm: hidden=%d", hidden);
  DSP_REQUIRE(!(write_back && !delta), "dsp_rmsnorm: write_back without delta");
  DSP_REQUIRE(dtype == DSP_F32 || dtype == DSP_BF16, "dsp_rmsnorm: unknown dtype %d", dtype);
  const bool fast = dtype == DSP_F32
      ? launch_rmsnorm_vec<float>(x, delta, w, y, rows, n_rows, hidden, eps, write_back, stream)
      : launch_rmsnorm_vec<bf16>(x, delta, w, y, rows, n_rows, hidden, eps, write_back, stream);
  if (fast) {
    DSP_CHECK_LAUNCH("dsp_rmsnorm");
    return 0;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == DSP_F32)
    rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>((float*)x, (const float*)delta,
                                                          (const float*)w, (float*)y, rows, hidden,
                                                          eps, write_back);
  else
    rmsnorm_kernel<bf16><<<n_rows, threads, 0, stream>>>((bf16*)x, (const bf16*)delta,
                                                         (const bf16*)w, (bf16*)y, rows, hidden, eps,
                                                         write_back);
  DSP_CHECK_LAUNCH("dsp_rmsnorm");
  return 0;
}

// ------------------------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gate(t, i)) * up(t, i), silu(g) = g / (1 + exp(-g)), in 32-bit.
// block == 0: gu row = [all gates | all ups].  block == b > 0: gates and ups interleaved in blocks
// of b columns: gate(t, i) at column (i / b) * 2b + i % b, up(t, i) b columns further.
__device__ __forceinline__ size_t gate_column(int i, int inter, int block) {
  return block ? (size_t)(i / block) * 2 * block + i % block : (size_t)i;
}
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int block) {
  const size_t t = blockIdx.x;
  const T* row = gu + t * 2 * (size_t)inter;
  const int up_off = block ? block : inter;
  T* o = out + t * (size_t)inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    const size_t gc = gate_column(i, inter, block);
    const float gv = to_f32(row[gc]);
    const float uv = to_f32(row[gc + up_off]);
    o[i] = from_f32<T>(gv / (1.f + expf(-gv)) * uv);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total_vecs,
                  int block) {
  constexpr int N = Vec16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = inter / N;
  const int up_off = block ? block : inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / vec_per_row;
    const int c = (int)(i % vec_per_row);
    const T* gp = gu + t * 2 * (size_t)inter + gate_column(c * N, inter, block);
    const uint4 graw = *reinterpret_cast<const uint4*>(gp);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gp + up_off);
    const T* g = reinterpret_cast<const T*>(&graw);
    const T* u = reinterpret_cast<const T*>(&uraw);
    uint4 oraw;
    T* o = reinterpret_cast<T*>(&oraw);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float gv = to_f32(g[k]);
      o[k] = from_f32<T>(gv / (1.f + expf(-gv)) * to_f32(u[k]));
    }
    reinterpret_cast<uint4*>(out + t * (size_t)inter)[c] = oraw;
  }
}

extern "C" int dsp_swiglu(const void* gate_up, void* out, int T, int inter, int block, int dtype,
                          cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(block >= 0 && (block == 0 || inter % block == 0),
              "dsp_swiglu: interleave block %d does not divide %d", block, inter);
  DSP_REQUIRE(dtype == DSP_F32 || dtype == DSP_BF16, "dsp_swiglu: unknown dtype %d", dtype);
  const int N = dtype == DSP_F32 ? 4 : 8;
  if (inter % N == 0 && (block == 0 || block % N == 0) && ((uintptr_t)gate_up % 16) == 0 &&
      ((uintptr_t)out % 16) == 0) {
    const size_t total = (size_t)T * (inter / N);
    const size_t cap = (size_t)(dsp_num_sms() > 0 ? dsp_num_sms() : 1) * 16;  // grid-stride loop beyond that
    const int blocks = (int)((total + 255) / 256 > cap ? cap : (total + 255) / 256);
    if (dtype == DSP_F32)
      launch_pdl(swiglu_vec_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, inter, total, block);
    else
      launch_pdl(swiglu_vec_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total, block);
    DSP_CHECK_LAUNCH("dsp_swiglu");
    return 0;
  }
  const int chunks = (inter + 255) / 256;
  dim3 grid(T, chunks > 64 ? 64 : chunks);
  if (dtype == DSP_F32)
    swiglu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, block);
  else
    swiglu_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, inter, block);
  DSP_CHECK_LAUNCH("dsp_swiglu");
  return 0;
}

// ------------------------------------------------- rotary encoding + paged key/value write
// qkv: [T, (H + 2*KVH) * D], heads in the order q..., k..., v....  One block per (token, head).
//  q head: rotated in place.
//  k head: rotated and written to k_pool[page, kvh, offset, :]  (also rotated in place).
//  v head: copied to v_pool[page, kvh, offset, :].
// The rotation pairs element i with i + rotary_dim/2 (half-split), angle = pos * inv_freq[i]
// in 32-bit: out[i] = x[i] cos - x[i+h] sin, out[i+h] = x[i+h] cos + x[i] sin.  Elements at
// and beyond rotary_dim pass through.  rotary_dim == 0 means no rotation at all.
// Pool layout: [num_pages, KVH, page_size, D].  page = page_table[seq, pos / page_size].
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int pt_stride,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const float* __restrict__ inv_freq, int H, int KVH, int D,
                                     int rotary_dim, int page_size, int num_pages, int write_kv,
                                     int* err) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;
  const int pos = positions[t];
  if (pos < 0) return;  // padding row of a fixed-shape batch
  T* x = qkv + ((size_t)t * (H + 2 * KVH) + head) * D;
  const bool is_q = head < H;
  const bool is_k = !is_q && head < H + KVH;
  T* dst = nullptr;
  if (!is_q) {
    if (!write_kv) return;
    const int seq = seq_of_token[t];
    const int page = page_table[(size_t)seq * pt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
      return;
    }
    const int kvh = is_k ? head - H : head - H - KVH;
    T* pool = is_k ? k_pool : v_pool;
    dst = pool + (((size_t)page * KVH + kvh) * page_size + (pos % page_size)) * D;
  }
  if (is_q || is_k) {
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float ang = (float)pos * inv_freq[i];
      float s, c;
      sincosf(ang, &s, &c);
      const float a = to_f32(x[i]), b = to_f32(x[i + half]);
      const T ra = from_f32<T>(a * c - b * s);
      const T rb = from_f32<T>(b * c + a * s);
      x[i] = ra;
      x[i + half] = rb;
      if (dst) {
        dst[i] = ra;
        dst[i + half] = rb;
      }
    }
    if (dst)
      for (int i = rotary_dim + threadIdx.x; i < D; i += blockDim.x) dst[i] = x[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = x[i];
  }
}

// One block per token for head sizes in whole 16-byte pieces: cos and sin of the token's angles
// are computed once into shared memory and every head reuses them; data moves in 16-byte pieces.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_store_token_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                           const int* __restrict__ seq_of_token,
                           const int* __restrict__ page_table, int pt_stride,
                           T* __restrict__ k_pool, T* __restrict__ v_pool,
                           const float* __restrict__ inv_freq, int H, int KVH, int D,
                           int rotary_dim, int page_size, int num_pages, int write_kv, int* err) {
  constexpr int N = Vec16<T>::N;
  extern __shared__ float cs[];  // cos[half], sin[half]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int half = rotary_dim / 2;
  // a thread's first pair of pieces is asked for before the angles are worked out, so that the
  // loads do not wait behind the sines, the cosines and the barrier
  T* const row0 = qkv + (size_t)t * (H + 2 * KVH) * D;
  const int hv0 = half / N;
  uint4 first_lo = make_uint4(0u, 0u, 0u, 0u), first_hi = first_lo;
  if ((int)threadIdx.x < (H + KVH) * hv0) {
    const int head = threadIdx.x / hv0, j = threadIdx.x % hv0;
    first_lo = reinterpret_cast<const uint4*>(row0 + (size_t)head * D)[j];
    first_hi = reinterpret_cast<const uint4*>(row0 + (size_t)head * D + half)[j];
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  long kv_base = -1;  // element offset of this token's row of kv head 0 in the pools
  if (write_kv) {
    const int seq = seq_of_token[t];
    const int page = page_table[(size_t)seq * pt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
    } else {
      kv_base = ((long)page * KVH * page_size + (pos % page_size)) * D;
    }
  }
  __syncthreads();
  T* row = qkv + (size_t)t * (H + 2 * KVH) * D;
  const int hv = half / N;        // 16-byte pieces in the rotated half
  const int dv = D / N;           // pieces per head
  // rotated heads (q and k): one work item rotates piece j of the low half with piece j of the high half
  const int rot_items = (H + KVH) * hv;
  for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
    const int head = it / hv, j = it % hv;
    uint4* lo_p = reinterpret_cast<uint4*>(row + (size_t)head * D) + j;
    uint4* hi_p = reinterpret_cast<uint4*>(row + (size_t)head * D + half) + j;
    uint4 lo, hi;
    if (it == (int)threadIdx.x) {
      lo = first_lo;
      hi = first_hi;
    } else {
      lo = *lo_p;
      hi = *hi_p;
    }
    T* a = reinterpret_cast<T*>(&lo);
    T* b = reinterpret_cast<T*>(&hi);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float c = cs[j * N + k], sn = cs[half + j * N + k];
      const float av = to_f32(a[k]), bv = to_f32(b[k]);
      a[k] = from_f32<T>(av * c - bv * sn);
      b[k] = from_f32<T>(bv * c + av * sn);
    }
    *lo_p = lo;
    *hi_p = hi;
    if (head >= H && kv_base >= 0) {
      T* dst = k_pool + kv_base + (long)(head - H) * page_size * D;
      reinterpret_cast<uint4*>(dst)[j] = lo;
      reinterpret_cast<uint4*>(dst + half)[j] = hi;
    }
  }
  if (kv_base < 0) return;
  // unrotated tail of k heads, and v heads
  const int tail_v = (D - rotary_dim) / N;
  for (int it = threadIdx.x; it < KVH * tail_v; it += blockDim.x) {
    const int kvh = it / tail_v, j = it % tail_v;
    const uint4 v = reinterpret_cast<const uint4*>(row + (size_t)(H + kvh) * D + rotary_dim)[j];
    reinterpret_cast<uint4*>(k_pool + kv_base + (long)kvh * page_size * D + rotary_dim)[j] = v;
  }
  for (int it = threadIdx.x; it < KVH * dv; it += blockDim.x) {
    const int kvh = it / dv, j = it % dv;
    const uint4 v = reinterpret_cast<const uint4*>(row + (size_t)(H + KVH + kvh) * D)[j];
    reinterpret_cast<uint4*>(v_pool + kv_base + (long)kvh * page_size * D)[j] = v;
  }
}

extern "C" int dsp_rope_kv_store(void* qkv, const int* positions, const int* seq_of_token,
                                 const int* page_table, int pt_stride, void* k_pool, void* v_pool,
                                 const float* inv_freq, int T, int H, int KVH, int D,
                                 int rotary_dim, int page_size, int num_pages, int write_kv,
                                 int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 2 == 0,
              "dsp_rope_kv_store: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, D);
  DSP_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "dsp_rope_kv_store: no inv_freq table");
  DSP_REQUIRE(H + 2 * KVH <= 65535, "dsp_rope_kv_store: too many heads");
  DSP_REQUIRE(dtype == DSP_F32 || dtype == DSP_BF16, "dsp_rope_kv_store: unknown dtype %d", dtype);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_rope_kv_store: no device error word");
  const int N = dtype == DSP_F32 ? 4 : 8;
  const uintptr_t bits = (uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool;
  if (rotary_dim > 0 && (rotary_dim / 2) % N == 0 && D % N == 0 && bits % 16 == 0 && rotary_dim <= 4096) {
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    const int threads = (H + KVH) * (rotary_dim / 2 / N) >= 256 ? 256 : 128;
    if (dtype == DSP_F32)
      DSP_CUDA(launch_pdl(rope_kv_store_token_kernel<float>, dim3(T), dim3(threads), smem, stream,
                          (float*)qkv, positions, seq_of_token, page_table, pt_stride, (float*)k_pool,
                          (float*)v_pool, inv_freq, H, KVH, D, rotary_dim, page_size, num_pages,
                          write_kv, err));
    else
      DSP_CUDA(launch_pdl(rope_kv_store_token_kernel<bf16>, dim3(T), dim3(threads), smem, stream,
                          (bf16*)qkv, positions, seq_of_token, page_table, pt_stride, (bf16*)k_pool,
                          (bf16*)v_pool, inv_freq, H, KVH, D, rotary_dim, page_size, num_pages,
                          write_kv, err));
    DSP_CHECK_LAUNCH("dsp_rope_kv_store");
    return 0;
  }
  dim3 grid(T, H + 2 * KVH);
  const int threads = D / 2 >= 64 ? 64 : 32;
  if (dtype == DSP_F32)
    rope_kv_store_kernel<float><<<grid, threads, 0, stream>>>(
        (float*)qkv, positions, seq_of_token, page_table, pt_stride, (float*)k_pool, (float*)v_pool,
        inv_freq, H, KVH, D, rotary_dim, page_size, num_pages, write_kv, err);
  else
    rope_kv_store_kernel<bf16><<<grid, threads, 0, stream>>>(
        (bf16*)qkv, positions, seq_of_token, page_table, pt_stride, (bf16*)k_pool, (bf16*)v_pool,
        inv_freq, H, KVH, D, rotary_dim, page_size, num_pages, write_kv, err);
  DSP_CHECK_LAUNCH("dsp_rope_kv_store");
  return 0;
}
