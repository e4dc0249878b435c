// Shared helpers of the kernel library: storage types, error reporting, reductions.
//
// The library has a C ABI over raw device pointers.  Every entry point returns 0 on
// success; otherwise dsp_last_error() holds a message.  Kernels never trap: a bad index
// (page id, token id) is skipped and recorded in a device error word that the host reads
// with dsp_device_error().
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

enum DspDtype { DSP_F32 = 0, DSP_BF16 = 1 };

// device error word bits
enum DspDeviceError {
  DSP_ERR_BAD_PAGE = 1,    // page id outside the pool
  DSP_ERR_BAD_TOKEN = 2,   // token id outside the vocabulary
  DSP_ERR_WAIT_LIMIT = 4,  // a bounded wait on a barrier ran out
};

extern "C" const char* dsp_last_error();
void dsp_set_error(const char* fmt, ...);
int* dsp_device_error_ptr();  // device address of the error word (per current device)
int dsp_num_sms();            // streaming multiprocessors of the current device (0 if unknown)

#define DSP_REQUIRE(cond, ...)  \
  do {                          \
    if (!(cond)) {              \
      dsp_set_error(__VA_ARGS__); \
      return 2;                 \
    }                           \
  } while (0)

#define DSP_CHECK_LAUNCH(name)                                   \
  do {                                                           \
    cudaError_t e__ = cudaGetLastError();                        \
    if (e__ != cudaSuccess) {                                    \
      dsp_set_error("%s: %s", name, cudaGetErrorString(e__));    \
      return 1;                                                  \
    }                                                            \
  } while (0)

#define DSP_CUDA(call)                                                        \
  do {                                                                        \
    cudaError_t e__ = (call);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      dsp_set_error("%s failed: %s", #call, cudaGetErrorString(e__));         \
      return 1;                                                               \
    }                                                                         \
  } while (0)

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the kernel
// before it in the stream is still running; it must call pdl_wait() before it touches anything
// that kernel (or any earlier one) wrote, and before it writes anything itself.  What it does
// before that (fetching weights, computing addresses) overlaps the tail of its predecessor.
// pdl_launch_dependents() lets the next kernel's launch begin.  Without the launch attribute
// both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// DISPEC_B200_PDL=0 in the environment switches the launch attribute off (for measurements).
inline bool pdl_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* v = getenv("DISPEC_B200_PDL");
    state = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return state == 1;
}

// Asks, once per kernel, for the largest shared-memory carveout.  The kernels of a step differ
// widely in the shared memory they use; with one carveout for all of them the SMs are not
// reconfigured between consecutive kernels.
inline void prefer_max_shared(const void* kernel) {
  static const void* seen[128];
  static int count = 0;
  for (int i = 0; i < count; ++i)
    if (seen[i] == kernel) return;
  if (count < 128) seen[count++] = kernel;
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum in a fixed order (lanes by xor tree, then warps in index order).
// `scratch` holds at least 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = -INFINITY;
  for (int w = 0; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
  return total;
}
