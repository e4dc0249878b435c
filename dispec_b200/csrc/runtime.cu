// Error reporting and the device error word.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[1024] = "";

void dsp_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* dsp_last_error() { return g_error; }

__device__ int g_dsp_device_error = 0;

int* dsp_device_error_ptr() {
  // looked up once per device (the lookup is not repeated under graph capture)
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_dsp_device_error) != cudaSuccess) return nullptr;
    cached[dev] = p;
  }
  return cached[dev];
}

int dsp_num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// Reads and clears the device error word (synchronises the device).
extern "C" int dsp_device_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dsp_device_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_dsp_device_error, &zero, sizeof(int));
  }
  return v;
}

extern "C" int dsp_abi_version() { return 1; }

// Device address of the error word, for kernels that live in other libraries.
extern "C" unsigned long long dsp_device_error_address() {
  return (unsigned long long)(uintptr_t)dsp_device_error_ptr();
}
