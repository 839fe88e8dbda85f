// Allocation-free arg-max entry point.
//
// This entry point has no counterpart in the reference plugin: it exists for callers of this
// library that are not allowed to allocate device memory at the point of the call - code running
// inside a fixed, pre-planned memory budget (an embedding runtime that hands the library raw
// pointers and owns every byte on the device), and callers that sit between cudaMalloc-free
// phases such as a real-time decode loop where an allocation could stall on the driver's lock.
// Everything else in the library may grow persistent scratch through the framework's allocator;
// this function never does.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of rows one call accepts.  The scratch behind it is a file-scope device array of
// B200_ARGMAX_NOALLOC_MAX_ROWS * 32 partial (value, index) pairs = 512 KiB, resident on every GPU
// that loads the library until the process exits.
#define B200_ARGMAX_NOALLOC_MAX_ROWS 2048

// out[r] = index of the largest element of logits[r, 0..V)  (ties -> lowest index), r < rows.
//   logits  device pointer, row stride `stride` elements, dtype 0 = f32, 1 = bf16, 2 = f16
//   out     device pointer to `rows` int64
// Returns 0 on success (rows == 0 is a successful no-op); 22 (EINVAL), with nothing launched, when
// rows > B200_ARGMAX_NOALLOC_MAX_ROWS, rows < 0, V <= 0, stride < V, dtype is not 0 / 1 / 2, or a pointer is
// null; otherwise the cudaError_t of the failing call.
//
// * Calls no cudaMalloc / cudaFree and no allocating library routine; the caller passes only its
//   inputs and outputs.
// * The first call on each device resolves the device address of the scratch array
//   (cudaGetSymbolAddress, with that device current) and caches it in a host-side table without a
//   lock.  Make that first call outside any stream capture, and do not let two host threads make
//   the first call on the same device at the same time (later calls only read the table).
// * All calls on one device share the one scratch array.  Each call overwrites every scratch
//   entry it later reads, so nothing needs clearing between calls - but two calls whose kernels
//   overlap on the GPU (different streams, no dependency) race on it.  Serialise them.
int b200_argmax_noalloc(int64_t* out, const void* logits, int64_t rows, int V, int64_t stride, int dtype,
                        cudaStream_t st);

#ifdef __cplusplus
}
#endif
