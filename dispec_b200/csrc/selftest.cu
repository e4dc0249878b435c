// Self-test entry points: they exercise the kernels' own error reporting in forms that cannot touch
// bad memory and cannot wait without bound.
#include "tcgen05_common.cuh"

namespace {
// One warp waits, with the product kernels' own bounded wait, on an mbarrier at which nothing ever
// arrives.  The wait runs out after `tries` tries, the kernel records DSP_ERR_WAIT_LIMIT in the
// device error word and returns normally: the context stays usable.
__global__ void wait_limit_kernel(uint32_t tries, int* err, int* ran_out) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool done = tc::mbar_wait_limit(&bar, 0, tries);
  if (!done && threadIdx.x == 0) {
    atomicOr(err, DSP_ERR_WAIT_LIMIT);
    *ran_out = 1;
  }
}
}  // namespace

// tries: at most 65,536 (each try blocks for a short, hardware-bounded time).  ran_out: a device
// int that is set to 1 when the wait ran out.
extern "C" int dsp_selftest_wait_limit(int tries, int* ran_out, cudaStream_t stream) {
  DSP_REQUIRE(tries > 0 && tries <= 65536, "dsp_selftest_wait_limit: tries=%d outside 1..65536", tries);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr && ran_out != nullptr, "dsp_selftest_wait_limit: no device error word or result");
  wait_limit_kernel<<<1, 32, 0, stream>>>((uint32_t)tries, err, ran_out);
  DSP_CHECK_LAUNCH("dsp_selftest_wait_limit");
  return 0;
}

// ---- how often one thread can issue tcgen05.mma --------------------------------------------------
// A measurement, kept with the library because the weight-streaming product is laid out by its result: `issuers` threads
// of different warps each issue `iters` products of 128 x n x 16 (bfloat16, operands resident in
// shared memory, an accumulator of its own each) and report the cycles per product of the first.
namespace {
__global__ void __launch_bounds__(128, 1) mma_issue_rate_kernel(int n, int iters, int issuers, long long* out) {
  using namespace tc;
  extern __shared__ unsigned char rate_smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rate_smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, issuers);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if ((threadIdx.x & 31) == 0 && warp < issuers) {
    const uint32_t idesc = umma_idesc(128, n);
    const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 16384);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma(tmem_base + (uint32_t)(warp * 128), umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, i > 0 || k > 0);
    }
    const long long t1 = clock64();
    umma_commit(&bar);
    const bool ok = mbar_wait(&bar, 0);  // bounded
    const long long t2 = clock64();
    if (warp == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      out[2] = ok ? 1 : 0;
    }
  }
  __syncthreads();
  tc_fence_after();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}
}  // namespace

// out: three device integers (64-bit): cycles until the first issuer's last product was issued, cycles
// until all products had completed, and 1 if the bounded wait for them returned in time.
// n: 16..128 in steps of 16; issuers: 1..4; iters: k blocks of four products each, at most 4096.
extern "C" int dsp_selftest_mma_issue_rate(int n, int issuers, int iters, long long* out, cudaStream_t stream) {
  DSP_REQUIRE(n >= 16 && n <= 128 && n % 16 == 0, "dsp_selftest_mma_issue_rate: n=%d outside 16..128 in steps of 16", n);
  DSP_REQUIRE(issuers >= 1 && issuers <= 4 && iters >= 1 && iters <= 4096 && out != nullptr,
              "dsp_selftest_mma_issue_rate: issuers=%d or iters=%d out of range", issuers, iters);
  static bool configured = false;
  if (!configured) {
    DSP_CUDA(cudaFuncSetAttribute(mma_issue_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    configured = true;
  }
  mma_issue_rate_kernel<<<1, 128, 64 * 1024, stream>>>(n, iters, issuers, out);
  DSP_CHECK_LAUNCH("dsp_selftest_mma_issue_rate");
  return 0;
}

// ---- how fast one SM takes tiles in by TMA --------------------------------------------------------
// A measurement, kept with the library because the many-row product's ring is laid out by its
// result: every CTA (one per SM) runs a ring of `stages` slots; one thread requests `boxes` boxes
// per slot from a matrix of `rows` x 1536 bfloat16 that lies in the L2 (each box 64 of k by 128
// rows by `k_blocks` blocks of k, through the three-dimensional map of make_map_k_blocks), another
// waits for them and frees the slot; nothing is computed.  out[0]: cycles per slot (mean over the
// CTAs), out[1]: 1 if no wait ran out.
namespace {
constexpr int TMA_RATE_MAX_STAGES = 8, TMA_RATE_K = 1536;
__global__ void __launch_bounds__(64, 1) tma_rate_kernel(const __grid_constant__ CUtensorMap map, int rows, int stages,
                                                          int boxes, int k_blocks, int iters, long long* cycles, int* ok) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[TMA_RATE_MAX_STAGES], empty_bar[TMA_RATE_MAX_STAGES];
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int box_bytes = 128 * 128 * k_blocks;
  const int steps_per_row_tile = TMA_RATE_K / 64 / k_blocks, row_tiles = rows / 128;
  const long long t0 = clock64();
  if (threadIdx.x == 0) {
    int s = 0, phase = 0;
    for (int it = 0; it < iters; ++it) {
      if (it >= stages && !tc::mbar_wait(&empty_bar[s], (uint32_t)(phase ^ 1))) {
        *ok = 0;
        break;
      }
      tc::mbar_expect_tx(&full_bar[s], (uint32_t)(boxes * box_bytes));
      for (int b = 0; b < boxes; ++b) {
        const int tile = ((int)blockIdx.x * 7 + it / steps_per_row_tile * 3 + b * 5) % row_tiles;
        tc::tma_load_3d(smem + (s * boxes + b) * box_bytes, &map, &full_bar[s], 0, tile * 128, (it % steps_per_row_tile) * k_blocks);
      }
      if (++s == stages) s = 0, phase ^= 1;
    }
  } else if (threadIdx.x == 32) {
    int s = 0, phase = 0;
    for (int it = 0; it < iters; ++it) {
      if (!tc::mbar_wait(&full_bar[s], (uint32_t)phase)) {
        *ok = 0;
        break;
      }
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc::smem_u32(&empty_bar[s])) : "memory");
      if (++s == stages) s = 0, phase ^= 1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) cycles[blockIdx.x] = clock64() - t0;
}
}  // namespace

// matrix: rows x 1536 bfloat16 on the device (rows a multiple of 128); cycles: one value per CTA;
// ok: set to 0 if a wait ran out (the caller sets it to 1 first)
extern "C" int dsp_selftest_tma_rate(const void* matrix, int rows, int stages, int boxes, int k_blocks, int ctas, int iters,
                                     long long* cycles, int* ok, cudaStream_t stream) {
  DSP_REQUIRE(matrix != nullptr && cycles != nullptr && ok != nullptr && rows >= 128 && rows % 128 == 0,
              "dsp_selftest_tma_rate: a matrix of a multiple of 128 rows and result buffers are needed (rows=%d)", rows);
  DSP_REQUIRE(stages >= 1 && stages <= TMA_RATE_MAX_STAGES && boxes >= 1 && boxes <= 8 && k_blocks >= 1 && k_blocks <= 8 &&
                  (TMA_RATE_K / 64) % k_blocks == 0 && ctas >= 1 && ctas <= 1024 && iters >= 1,
              "dsp_selftest_tma_rate: stages=%d, boxes=%d or k_blocks=%d out of range", stages, boxes, k_blocks);
  const size_t smem = (size_t)stages * boxes * 128 * 128 * k_blocks + 1024;
  DSP_REQUIRE(smem <= 227 * 1024, "dsp_selftest_tma_rate: %zu bytes of shared memory asked for", smem);
  CUtensorMap map;
  DSP_REQUIRE(tc::make_map_k_blocks(&map, matrix, rows, TMA_RATE_K, TMA_RATE_K, 128, k_blocks),
              "dsp_selftest_tma_rate: cannot encode the tensor map");
  DSP_CUDA(cudaFuncSetAttribute(tma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  tma_rate_kernel<<<ctas, 64, smem, stream>>>(map, rows, stages, boxes, k_blocks, iters, cycles, ok);
  DSP_CHECK_LAUNCH("dsp_selftest_tma_rate");
  return 0;
}
