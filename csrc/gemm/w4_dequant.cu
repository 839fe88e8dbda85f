// 4-bit weights (AWQ / GPTQ after repacking) -> a 16-bit [N, K] matrix, for batches too large for the decode kernel:
// the bf16 GEMM then runs on the temporary.  (The reference de-quantises for 256 tokens and more and calls a fused
// kernel below that: vllm_kunlun/quantization/awq.py:124-168; `_C::awq_dequantize`, ops/_custom_ops.py:1416-1440.)
//
// Packed layout (quantization/int4.py::pack_w4): row n holds K / 2 bytes; the 32-bit word j of the row holds the k
// positions 8 j .. 8 j + 7 with their nibbles in the order 0, 2, 4, 6, 1, 3, 5, 7 - the order in which
// csrc/gemm/gemm_decode.cu extracts pairs.  scale / zero: [N, K / group] in the output type.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/utils.cuh"

namespace b200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) dequant_w4_kernel(T* __restrict__ out, const uint32_t* __restrict__ packed,
                                                         const T* __restrict__ scale, const T* __restrict__ zero,
                                                         int64_t words, int words_per_row, int group) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= words) return;
  const int64_t n = i / words_per_row;
  const int j = (int)(i - n * words_per_row);
  const int groups = words_per_row * 8 / group;
  const int gi = (j * 8) / group;
  const float s = to_f(scale[n * groups + gi]), z = to_f(zero[n * groups + gi]);
  const uint32_t w = packed[i];
  alignas(16) T v[8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float lo = (float)((w >> (4 * p)) & 0xFu), hi = (float)((w >> (4 * p + 16)) & 0xFu);
    v[2 * p] = from_f<T>((lo - z) * s);
    v[2 * p + 1] = from_f<T>((hi - z) * s);
  }
  *reinterpret_cast<uint4*>(out + i * 8) = *reinterpret_cast<const uint4*>(v);
}

}  // namespace
}  // namespace b200

extern "C" int b200_dequant_w4(void* out, const void* packed, const void* scale, const void* zero, int64_t N, int K,
                               int group, int dtype, cudaStream_t st) {
  if (N == 0 || K == 0) return 0;
  if (K % 8 != 0 || group % 8 != 0 || K % group != 0 || dtype == 0) return 3;
  const int64_t words = N * (K / 8);
  const unsigned blocks = (unsigned)((words + 255) / 256);
  if (dtype == b200::kBF16)
    b200::dequant_w4_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)out, (const uint32_t*)packed,
                                                                   (const __nv_bfloat16*)scale, (const __nv_bfloat16*)zero,
                                                                   words, K / 8, group);
  else
    b200::dequant_w4_kernel<__half><<<blocks, 256, 0, st>>>((__half*)out, (const uint32_t*)packed, (const __half*)scale,
                                                            (const __half*)zero, words, K / 8, group);
  return cudaGetLastError() != cudaSuccess;
}
