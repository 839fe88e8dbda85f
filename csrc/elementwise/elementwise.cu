// Normalisation, activation, embedding and arg-max kernels (bandwidth-bound, 16-byte vector access,
// fp32 math).  Semantics follow the fp32 oracles in vllm_kunlun_b200/ops/reference/basic.py.
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

constexpr int kNormThreads = 256;
constexpr int kMaxCached = 4;  // 16-byte chunks kept in registers per thread

// out = rmsnorm(x [+ residual]) * w;  when residual != nullptr it is updated in place with the sum
// (rounded to T first, as the sum is what later layers read back).  `x` may alias `out`.
template <typename T, bool kAdd>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(T* __restrict__ out, const T* x, T* residual,
                                                               const T* __restrict__ w, int H, float eps, int gemma,
                                                               int64_t x_stride, int64_t out_stride) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  const T* xr = x + row * x_stride;
  T* rr = kAdd ? residual + row * (int64_t)H : nullptr;
  T* orow = out + row * out_stride;
  const int nvec = H / V;
  Vec16<T> cache[kMaxCached];
  float ss = 0.f;
  int c = 0;
  for (int i = threadIdx.x; i < nvec; i += kNormThreads, ++c) {
    Vec16<T> a = ld_vec(xr + i * V);
    if (kAdd) {
      Vec16<T> b = ld_vec(rr + i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) a.v[j] = from_f<T>(to_f(a.v[j]) + to_f(b.v[j]));
      st_vec(rr + i * V, a);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) { float f = to_f(a.v[j]); ss += f * f; }
    if (c < kMaxCached) cache[c] = a;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / H + eps);
  c = 0;
  for (int i = threadIdx.x; i < nvec; i += kNormThreads, ++c) {
    Vec16<T> a = (c < kMaxCached) ? cache[c] : ld_vec((kAdd ? (const T*)rr : xr) + i * V);
    Vec16<T> ww = ld_vec(w + i * V);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float g = to_f(ww.v[j]) + (gemma ? 1.f : 0.f);
      a.v[j] = from_f<T>(to_f(a.v[j]) * inv * g);
    }
    st_vec(orow + i * V, a);
  }
}

// Many short rows (per-head norms, l2norm, gated norm): one warp per row.
template <typename T, int kMode>  // 0 = rmsnorm*w, 1 = l2norm, 2 = gated (norm then *silu(z)), 3 = gated (silu first)
__global__ void warp_rownorm_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ z,
                                    const T* __restrict__ w, int64_t rows, int D, float eps, int w_period) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int lane = threadIdx.x & 31;
  const T* xr = x + row * D;
  const T* zr = (kMode >= 2) ? z + row * D : nullptr;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float f = to_f(xr[i]);
    if (kMode == 3) { float g = to_f(zr[i]); f *= g / (1.f + __expf(-g)); }
    ss += f * f;
  }
  ss = warp_sum(ss);
  float inv = (kMode == 1) ? rsqrtf(ss + eps) : rsqrtf(ss / D + eps);
  for (int i = lane; i < D; i += 32) {
    float f = to_f(xr[i]);
    if (kMode == 3) { float g = to_f(zr[i]); f *= g / (1.f + __expf(-g)); }
    f *= inv;
    if (kMode != 1) f *= to_f(w[i]);
    if (kMode == 2) { float g = to_f(zr[i]); f *= g / (1.f + __expf(-g)); }
    out[row * D + i] = from_f<T>(f);
  }
}

// act: 0 = silu(gate)*up with x = [gate | up]; 1 = gelu_tanh(gate)*up; 2 = swigluoai (interleaved, clamped)
template <typename T>
__global__ void act_and_mul_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int d, int act) {
  constexpr int V = Vec16<T>::N;
  griddep_launch();
  griddep_wait();
  const int nvec = d / V;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = rows * nvec;
  if (idx >= total) return;
  int64_t row = idx / nvec;
  int i = (int)(idx - row * nvec);
  const T* xr = x + row * 2 * (int64_t)d;
  Vec16<T> o;
  if (act == 2) {
    Vec16<T> a = ld_vec(xr + 2 * i * V), b = ld_vec(xr + 2 * i * V + V);
    float vals[2 * V];
#pragma unroll
    for (int j = 0; j < V; ++j) { vals[j] = to_f(a.v[j]); vals[V + j] = to_f(b.v[j]); }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float g = fminf(vals[2 * j], 7.0f);
      float u = fminf(fmaxf(vals[2 * j + 1], -7.0f), 7.0f);
      o.v[j] = from_f<T>((u + 1.f) * g / (1.f + __expf(-1.702f * g)));
    }
  } else {
    Vec16<T> g = ld_vec(xr + i * V), u = ld_vec(xr + d + i * V);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float gf = to_f(g.v[j]), uf = to_f(u.v[j]);
      float a;
      if (act == 0) a = gf / (1.f + __expf(-gf));
      else { float t = 0.7978845608f * (gf + 0.044715f * gf * gf * gf); a = 0.5f * gf * (1.f + tanhf(t)); }
      o.v[j] = from_f<T>(a * uf);
    }
  }
  st_vec(out + row * (int64_t)d + i * V, o);
}

template <typename T>
__global__ void quick_gelu_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { float f = to_f(x[i]); out[i] = from_f<T>(f / (1.f + __expf(-1.702f * f))); }
}

template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const int64_t* __restrict__ ids, const T* __restrict__ w,
                                 int H, int64_t rows, int64_t vocab_start) {
  constexpr int V = Vec16<T>::N;
  griddep_launch();
  griddep_wait();
  int64_t t = blockIdx.x;
  int64_t id = ids[t] - vocab_start;
  bool ok = id >= 0 && id < rows;
  const T* src = w + (ok ? id : 0) * H;
  for (int i = threadIdx.x; i < H / V; i += blockDim.x) {
    Vec16<T> a;
    if (ok) a = ld_vec(src + i * V);
    else {
#pragma unroll
      for (int j = 0; j < V; ++j) a.v[j] = from_f<T>(0.f);
    }
    st_vec(out + t * H + i * V, a);
  }
}

// Arg-max over the vocabulary, two stages: grid (rows, chunks) partial maxima with 16-byte loads,
// then one warp per row over the chunk results.  Ties resolve to the lowest index (torch.argmax).
__device__ __forceinline__ void argmax_combine(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

template <typename T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(float* __restrict__ pval, int* __restrict__ pidx,
                                                             const T* __restrict__ logits, int V_, int64_t stride,
                                                             int chunk) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float sv[8];
  __shared__ int si[8];
  griddep_launch();
  griddep_wait();
  const T* row = logits + blockIdx.x * stride;
  const int lo = blockIdx.y * chunk, hi = min(V_, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) && (lo % VN == 0);
  int i0 = lo;
  if (vec_ok) {
    const int nvec = (hi - lo) / VN;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec16<T> a = ld_vec(row + lo + v * VN);
#pragma unroll
      for (int j = 0; j < VN; ++j) argmax_combine(best, bi, to_f(a.v[j]), lo + v * VN + j);
    }
    i0 = lo + nvec * VN;
  }
  for (int i = i0 + threadIdx.x; i < hi; i += blockDim.x) argmax_combine(best, bi, to_f(row[i]), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffff, best, o), __shfl_xor_sync(0xffffffff, bi, o));
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    best = l < 8 ? sv[l] : -INFINITY;
    bi = l < 8 ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1)
      argmax_combine(best, bi, __shfl_xor_sync(0xffffffff, best, o), __shfl_xor_sync(0xffffffff, bi, o));
    if (l == 0) { pval[blockIdx.x * gridDim.y + blockIdx.y] = best; pidx[blockIdx.x * gridDim.y + blockIdx.y] = bi; }
  }
}

__global__ void argmax_final_kernel(int64_t* __restrict__ out, const float* __restrict__ pval,
                                    const int* __restrict__ pidx, int chunks) {
  griddep_launch();
  griddep_wait();
  const int row = blockIdx.x, l = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = l; c < chunks; c += 32) argmax_combine(best, bi, pval[row * chunks + c], pidx[row * chunks + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffff, best, o), __shfl_xor_sync(0xffffffff, bi, o));
  if (l == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rmsnorm(void* out, const void* x, void* residual, const void* w, int64_t rows, int H, float eps,
                            int gemma, int64_t x_stride, int64_t out_stride, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    if (H % Vec16<T>::N) return 2;
    if (residual)
      launch_pdl(rmsnorm_kernel<T, true>, dim3(rows), dim3(kNormThreads), 0, st, (T*)out, (const T*)x, (T*)residual,
                 (const T*)w, H, eps, gemma, x_stride, out_stride);
    else
      launch_pdl(rmsnorm_kernel<T, false>, dim3(rows), dim3(kNormThreads), 0, st, (T*)out, (const T*)x, (T*)nullptr,
                 (const T*)w, H, eps, gemma, x_stride, out_stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_rownorm(void* out, const void* x, const void* z, const void* w, int64_t rows, int D, float eps,
                            int mode, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  int wpb = 8;
  int64_t grid = (rows + wpb - 1) / wpb;
  B200_DISPATCH_DTYPE(dtype, {
    switch (mode) {
      case 0: warp_rownorm_kernel<T, 0><<<grid, wpb * 32, 0, st>>>((T*)out, (const T*)x, nullptr, (const T*)w, rows, D, eps, 1); break;
      case 1: warp_rownorm_kernel<T, 1><<<grid, wpb * 32, 0, st>>>((T*)out, (const T*)x, nullptr, nullptr, rows, D, eps, 1); break;
      case 2: warp_rownorm_kernel<T, 2><<<grid, wpb * 32, 0, st>>>((T*)out, (const T*)x, (const T*)z, (const T*)w, rows, D, eps, 1); break;
      default: warp_rownorm_kernel<T, 3><<<grid, wpb * 32, 0, st>>>((T*)out, (const T*)x, (const T*)z, (const T*)w, rows, D, eps, 1); break;
    }
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_act_and_mul(void* out, const void* x, int64_t rows, int d, int act, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    constexpr int V = Vec16<T>::N;
    if (d % V || (act == 2 && d % V)) return 2;
    int64_t total = rows * (d / V);
    launch_pdl(act_and_mul_kernel<T>, dim3((total + 255) / 256), dim3(256), 0, st, (T*)out, (const T*)x, rows, d, act);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_quick_gelu(void* out, const void* x, int64_t n, int dtype, cudaStream_t st) {
  if (n == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, { quick_gelu_kernel<T><<<(n + 255) / 256, 256, 0, st>>>((T*)out, (const T*)x, n); });
  return (int)cudaGetLastError();
}

extern "C" int b200_embedding(void* out, const int64_t* ids, const void* w, int64_t T_, int H, int64_t rows,
                              int64_t vocab_start, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    if (H % Vec16<T>::N) return 2;
    launch_pdl(embedding_kernel<T>, dim3(T_), dim3(128), 0, st, (T*)out, ids, (const T*)w, H, rows, vocab_start);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_argmax(int64_t* out, const void* logits, int64_t rows, int V_, int64_t stride, int dtype,
                           float* scratch_val, int* scratch_idx, int chunks, cudaStream_t st) {
  if (rows == 0) return 0;
  int chunk = ((V_ + chunks - 1) / chunks + 15) / 16 * 16;
  chunks = (V_ + chunk - 1) / chunk;
  B200_DISPATCH_DTYPE(dtype, {
    launch_pdl(argmax_partial_kernel<T>, dim3(rows, chunks), dim3(256), 0, st, scratch_val, scratch_idx,
               (const T*)logits, V_, stride, chunk);
  });
  launch_pdl(argmax_final_kernel, dim3(rows), dim3(32), 0, st, out, (const float*)scratch_val,
             (const int*)scratch_idx, chunks);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of b200_argmax (declaration and contract: no_alloc.h).
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

namespace {
constexpr int kNoAllocChunks = 32;
struct ArgmaxPartial { float val; int idx; };
// File-scope scratch: MAX_ROWS x 32 partial maxima, split into a value plane and an index plane.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_argmax_scratch[B200_ARGMAX_NOALLOC_MAX_ROWS * kNoAllocChunks *
                                                                 sizeof(ArgmaxPartial)];
constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int b200_argmax_noalloc(int64_t* out, const void* logits, int64_t rows, int V_, int64_t stride, int dtype,
                                   cudaStream_t st) {
  if (out == nullptr || logits == nullptr || rows < 0 || V_ <= 0 || rows > B200_ARGMAX_NOALLOC_MAX_ROWS) return 22;
  if (stride < V_ || dtype < 0 || dtype > 2) return 22;  // rows would overlap / unknown element type
  if (rows == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return 22;
  if (g_scratch_ptr[dev] == nullptr) {
    // once per device, with that device current: the device address of the file-scope array
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_argmax_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_ptr[dev] = p;
  }
  float* sval = reinterpret_cast<float*>(g_scratch_ptr[dev]);
  int* sidx = reinterpret_cast<int*>(sval + (size_t)B200_ARGMAX_NOALLOC_MAX_ROWS * kNoAllocChunks);
  return b200_argmax(out, logits, rows, V_, stride, dtype, sval, sidx, kNoAllocChunks, st);
}
