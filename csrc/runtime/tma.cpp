// Host-side TMA descriptor encoding.  cuTensorMapEncodeTiled is resolved through the runtime's
// driver-entry-point lookup, so the library does not link against libcuda directly.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include <mutex>

#include "../api.h"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

extern "C" int b200_encode_tmap_2d(void* out, const void* base, uint64_t rows, uint64_t cols,
                                   uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return 1001;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) return 1002;
  if ((uint64_t)box_cols * elem_bytes != 128 || box_rows > 256) return 1003;
  CUtensorMap tm;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(&tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 2000 + (int)r;
  memcpy(out, &tm, sizeof(tm));
  return 0;
}

extern "C" int b200_encode_tmap_2d_raw(void* out, const void* base, uint64_t rows, uint64_t row_bytes,
                                       uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_bytes) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return 1001;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) return 1002;
  if (box_bytes == 0 || (box_bytes & 15) || box_bytes > 256 || box_rows > 256) return 1003;
  CUtensorMap tm;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 2000 + (int)r;
  memcpy(out, &tm, sizeof(tm));
  return 0;
}

// ---- PDL switch (see common/launch.cuh) ----
#include <stdlib.h>

#include <map>
#include <mutex>
#include <utility>
namespace b200 {
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> done;  // (kernel, device) -> limit already set
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_pair(kernel, dev);
  auto it = done.find(key);
  if (it != done.end() && it->second >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[key] = bytes;
  return e;
}
int pdl_enabled() {
  static int v = [] {
    const char* e = getenv("B200_PDL");
    return (e != nullptr && e[0] == '0') ? 0 : 1;
  }();
  return v;
}
// k-blocks (16 KB weight tiles) per CTA that a decode-shaped GEMM pulls into L2 ahead of its shared-memory ring
// before it waits for the previous kernel.  Off by default: on Llama-3.1-8B decode steps (batch 16) a depth of 24
// raised the step time from 5.10 to 5.34 ms and 64 to 5.59 ms - the memory system is already busy across kernel
// boundaries through the ring prefetch, and the extra requests only add traffic.
int gemm_l2_prefetch() {
  static int v = [] {
    const char* e = getenv("B200_GEMM_L2_PREFETCH");
    int n = e != nullptr ? atoi(e) : 0;
    return n < 0 ? 0 : (n > 256 ? 256 : n);
  }();
  return v;
}
}  // namespace b200
