// Pieces shared by the tcgen05 GEMM kernels: bounded waits with a CTA-wide abort flag and
// float conversions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../common/ptx.cuh"

namespace b200 {

struct Abort {
  int* status;
  volatile int* flag;  // shared-memory abort flag
  __device__ __forceinline__ bool aborted() const { return *flag != 0; }
  __device__ __forceinline__ void raise(int code) {
    *flag = 1;
    atomicCAS(status, 0, code);
  }
};

// Bounded wait that also leaves early once another role of this CTA has given up.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Abort& ab, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < (1u << 20); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && ab.aborted()) return false;
  }
  ab.raise(code);
  return false;
}

template <typename OutT>
__device__ __forceinline__ OutT from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half(v); }
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

}  // namespace b200
