// Multi-adapter LoRA kernels: shrink (x @ A[id]^T * scale -> fp32 [T, r]) and expand
// (out[:, off:off+N] (+)= h @ B[id]^T), with the adapter chosen per token.  Segment-wise calls (one adapter
// per sequence, prefill) and per-token calls (decode) share the kernels: segments are expanded to a per-token
// id vector by the caller.
//
// Reference entry points: _C::sgmv_shrink_lora / sgmv_expand(_slice)_lora / bgmv_shrink_lora /
// bgmv_expand(_slice)_lora (vllm_kunlun/ops/_custom_ops.py:2435-2836), driven by PunicaWrapperKunlun
// (vllm_kunlun/lora/punica_wrapper/punica_kunlun.py:273-545).
#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {
namespace {

// One block per token: the activation row is staged in shared memory once, each warp produces rank rows.
template <typename T>
__global__ void __launch_bounds__(256) lora_shrink_kernel(float* __restrict__ out, const T* __restrict__ x, int64_t x_stride,
                                                          const T* __restrict__ A /*[L, r, K]*/, const int* __restrict__ ids,
                                                          int r, int K, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sx = reinterpret_cast<T*>(smem_raw);
  const int64_t t = blockIdx.x;
  const int id = ids[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (id < 0) {
    for (int j = threadIdx.x; j < r; j += blockDim.x) out[t * r + j] = 0.f;
    return;
  }
  constexpr int VN = Vec16<T>::N;
  for (int i = threadIdx.x * VN; i < K; i += blockDim.x * VN) st_vec(sx + i, ld_vec(x + t * x_stride + i));
  __syncthreads();
  for (int j = warp; j < r; j += nw) {
    const T* a = A + ((int64_t)id * r + j) * K;
    float acc = 0.f;
    for (int i = lane * VN; i < K; i += 32 * VN) {
      Vec16<T> av = ld_vec(a + i), xv = ld_vec(sx + i);
#pragma unroll
      for (int e = 0; e < VN; ++e) acc += to_f(av.v[e]) * to_f(xv.v[e]);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[t * r + j] = acc * scale;
  }
}

// grid (T, ceil(N / 256)): one thread per output column; h row (r fp32) in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) lora_expand_kernel(T* __restrict__ out, int64_t out_stride, int offset,
                                                          const float* __restrict__ h, const T* __restrict__ B /*[L, N, r]*/,
                                                          const int* __restrict__ ids, int N, int r, int add) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sh = reinterpret_cast<float*>(smem_raw);
  const int64_t t = blockIdx.x;
  const int id = ids[t];
  if (id < 0) return;
  for (int j = threadIdx.x; j < r; j += blockDim.x) sh[j] = h[t * r + j];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const T* b = B + ((int64_t)id * N + n) * r;
  float acc = 0.f;
  constexpr int VN = Vec16<T>::N;
  if (r % VN == 0) {
    for (int j = 0; j < r; j += VN) {
      Vec16<T> bv = ld_vec(b + j);
#pragma unroll
      for (int e = 0; e < VN; ++e) acc += to_f(bv.v[e]) * sh[j + e];
    }
  } else {
    for (int j = 0; j < r; ++j) acc += to_f(b[j]) * sh[j];
  }
  T* o = out + t * out_stride + offset + n;
  *o = from_f<T>(add ? to_f(*o) + acc : acc);
}

}  // namespace
}  // namespace b200

extern "C" int b200_lora_shrink(float* out, const void* x, int64_t x_stride, const void* A, const int* ids, int64_t T_, int r,
                                int K, float scale, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  int esz = dtype == 0 ? 4 : 2;
  if (K % (16 / esz) != 0 || (x_stride * esz) % 16 != 0) return 3;
  size_t smem = (size_t)K * esz;
  if (smem > 200 * 1024) return 3;
  B200_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024) b200::ensure_dynamic_smem((const void*)b200::lora_shrink_kernel<T>, (int)smem);
    b200::lora_shrink_kernel<T><<<(unsigned)T_, 256, smem, st>>>(out, (const T*)x, x_stride, (const T*)A, ids, r, K, scale);
  });
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_lora_expand(void* out, int64_t out_stride, int offset, const float* h, const void* B, const int* ids,
                                int64_t T_, int N, int r, int add, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  dim3 grid((unsigned)T_, (N + 255) / 256);
  B200_DISPATCH_DTYPE(dtype, (b200::lora_expand_kernel<T><<<grid, 256, (size_t)r * 4, st>>>((T*)out, out_stride, offset, h,
                                                                                           (const T*)B, ids, N, r, add)));
  return cudaGetLastError() != cudaSuccess;
}
