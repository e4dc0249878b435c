/* Entry point for callers that cannot allocate device memory.
 *
 * This has no counterpart in the reference engine (puneethgv/DiSpec has no native code and
 * leaves all device memory to its tensor library).
 *
 * Who needs it: a program that drives the kernels through the C ABI from a place where
 * cudaMalloc is off limits.  Typical cases are a host application that hands the whole device
 * to an arena of its own at start-up and forbids later driver allocations, a latency-critical
 * loop that cannot afford the device-wide synchronisation an allocation may imply, and a
 * plug-in that has no access to the tensor library whose caching allocator the Python layer of
 * this package leans on.  The ordinary argmax entry point (dsp_argmax) expects such callers to
 * bring scratch memory for its two-stage form; this one brings its own.
 *
 * dsp_argmax_static(logits, stride, n, V, out, stream)
 *   out[r] = index of the largest of logits[r * stride .. + V), ties to the lowest index,
 *   for r < n; int32 output, float32 input, both on the device, launched on `stream`.
 *   Returns 0, or non-zero with a message in dsp_last_error().
 *
 * Scratch: the per-chunk partial results live in one array that is part of the library image
 * (static __device__, 512 KiB: 1024 rows x 64 chunks x 8 bytes).  Every device that loads the
 * library holds that array until the process exits.  Calls with more than
 * dsp_argmax_static_max_rows() rows are refused.  The entry point calls neither cudaMalloc nor
 * cudaFree nor any routine that allocates.
 *
 * First call on a device: it looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) and keeps it.  Make that first call outside any stream capture.  Several
 * host threads may make their first call on a device at the same time: each looks the same
 * address up and stores the same value, no lock is needed.
 *
 * Sharing: all calls on a device use the same array, and it keeps the previous call's
 * contents.  Nothing in it has to start at zero: every slot a call reads was written by that
 * same call first.  Two calls that overlap in time on the device (different streams) race on
 * it; serialise them.
 */
#ifndef DISPEC_B200_NO_ALLOC_H
#define DISPEC_B200_NO_ALLOC_H

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

int dsp_argmax_static(const float* logits, long stride, int n, int V, int* out, cudaStream_t stream);
int dsp_argmax_static_max_rows(void);

#ifdef __cplusplus
}
#endif

#endif
