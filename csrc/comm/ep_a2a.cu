// Expert-parallel dispatch / combine over NVLink peer memory.
//
// Every rank owns its own tokens (sequence- or data-parallel layout) and E / R whole experts.  The reference
// has no all-to-all: with expert parallelism it replicates all tokens on all ranks, loops over local experts in
// Python and lets the layer's all-reduce combine the result (KunlunOps.fused_moe_ep,
// vllm_kunlun/ops/_kunlun_ops.py:639-696; call site C6 models/deepseek_v2.py:303-306).  Here:
//
//   dispatch_send   one warp per local token: for every rank that owns at least one of the token's top-k experts
//                   (a token travels to a rank once, however many of its experts live there) claim a slot in that
//                   rank's receive region [source][slot] and write the payload row (bf16, or fp8 + 1x128 scales),
//                   the local expert ids (-1 for experts elsewhere) and the routing weights with 16-byte peer
//                   stores.  The last CTA publishes (epoch, count) to every destination with one release store.
//   dispatch_wait   on the receiving side: bounded wait for all R sources, counts to device memory, ids of the
//                   unused rows of every source region are invalidated.
//   (local)         permute by expert -> grouped GEMM -> activation -> grouped GEMM over the received rows.
//   combine_send    one CTA per received row: weighted sum of the row's local expert outputs, stored straight into
//                   the source rank's combine buffer [expert rank][slot]; the last CTA raises the flags.
//   combine_recv    on the source: bounded wait for all R expert ranks, then out[t] = sum over the ranks the token
//                   went to, in rank order (deterministic), plus an optional addend (shared experts).
//
// Buffer reuse needs no extra barrier: a source starts the next dispatch only after combine_recv has seen the
// flags of all expert ranks, and an expert rank raises its flag only after its last read of the receive region.
// All flags carry a call epoch kept in device memory (advanced by combine_recv), so the sequence can be replayed
// from a CUDA graph.  No NVLS multicast, no bulk-tensor copies: plain ld / st with .sys scope.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/utils.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ void st_release_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) ep_dispatch_send_kernel(EpArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const uint32_t epoch = *a.epoch + 1;
  const int e_loc = a.E / a.R;
  const int ngroups = a.H / 128;
  for (int64_t t = (int64_t)blockIdx.x * wpb + warp; t < a.T; t += (int64_t)gridDim.x * wpb) {
    const int* ids = a.topk_ids + t * a.k;
    const float* wts = a.topk_w + t * a.k;
    for (int d = 0; d < a.R; ++d) {
      bool hit = false;
      for (int j = 0; j < a.k; ++j) {
        int e = ids[j];
        hit |= (e >= 0 && e / e_loc == d);
      }
      int slot = -1;
      if (hit) {
        if (lane == 0) slot = atomicAdd(&a.send_count[d], 1);
        slot = __shfl_sync(0xffffffff, slot, 0);
        if (slot >= a.cap) { slot = -1; if (lane == 0) atomicCAS(a.status, 0, 410); }
      }
      if (lane == 0) a.sent_slot[t * a.R + d] = slot;
      if (slot < 0) continue;
      char* base = (char*)a.peer[d];
      const int64_t row = (int64_t)a.rank * a.cap + slot;
      // payload row
      const uint4* src = reinterpret_cast<const uint4*>((const char*)a.x + t * a.x_row_bytes);
      uint4* dst = reinterpret_cast<uint4*>(base + a.off_x + row * a.row_bytes);
      for (int i = lane; i < a.row_bytes / 16; i += 32) dst[i] = src[i];
      if (a.x_scale_t != nullptr) {  // fp8 payload: 1x128 scales, stored transposed [group][token] by the quantiser
        float* sd = reinterpret_cast<float*>(base + a.off_scale) + row * ngroups;
        for (int g = lane; g < ngroups; g += 32) sd[g] = a.x_scale_t[(int64_t)g * a.scale_stride + t];
      }
      if (lane < a.k) {
        int e = ids[lane];
        int le = (e >= 0 && e / e_loc == d) ? e - d * e_loc : -1;
        reinterpret_cast<int*>(base + a.off_ids)[row * a.k + lane] = le;
        reinterpret_cast<float*>(base + a.off_w)[row * a.k + lane] = wts[lane];
      }
    }
  }
  // publish: every CTA fences its peer stores, the last one to finish raises the flags
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < a.R) {
    const int d = threadIdx.x;
    int cnt = atomicAdd(&a.send_count[d], 0);
    if (cnt > a.cap) cnt = a.cap;
    uint64_t* flag = reinterpret_cast<uint64_t*>((char*)a.peer[d] + a.off_recv_flag) + a.rank;
    st_release_u64(flag, ((uint64_t)epoch << 32) | (uint32_t)cnt);
    a.send_count[d] = 0;
  }
  if (threadIdx.x == 0) *a.ticket = 0;
}

// grid = R CTAs (one per source)
__global__ void __launch_bounds__(256) ep_dispatch_wait_kernel(EpArgs a) {
  __shared__ int s_cnt;
  const int s = blockIdx.x;
  const uint32_t epoch = *a.epoch + 1;
  char* base = (char*)a.peer[a.rank];
  if (threadIdx.x == 0) {
    const uint64_t* flag = reinterpret_cast<const uint64_t*>(base + a.off_recv_flag) + s;
    int cnt = -1;
    for (uint32_t i = 0; i < a.spin_limit; ++i) {
      uint64_t v = ld_acquire_u64(flag);
      if ((uint32_t)(v >> 32) == epoch) { cnt = (int)(uint32_t)v; break; }
      if (i > 32) __nanosleep(64);
    }
    if (cnt < 0) { atomicCAS(a.status, 0, 420 + s); cnt = 0; }
    s_cnt = cnt;
    a.recv_count[s] = cnt;
  }
  __syncthreads();
  // rows of this source's region that carry nothing this call must read as "no local expert" (the region stride
  // is the per-call capacity, so rows of an earlier call with another capacity may be lying anywhere in it)
  const int cnt = s_cnt;
  int* ids = reinterpret_cast<int*>(base + a.off_ids) + ((int64_t)s * a.cap) * a.k;
  for (int i = cnt * a.k + threadIdx.x; i < a.cap * a.k; i += blockDim.x) ids[i] = -1;
}

// One CTA per row of the receive region.
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_send_kernel(EpArgs a, const T* __restrict__ y_sorted,
                                                              const int* __restrict__ pos_of_pair) {
  constexpr int V = Vec16<T>::N;
  const uint32_t epoch = *a.epoch + 1;
  const int64_t row = blockIdx.x;
  const int s = (int)(row / a.cap), slot = (int)(row % a.cap);
  char* mine = (char*)a.peer[a.rank];
  if (slot < a.recv_count[s]) {
    const float* w = reinterpret_cast<const float*>(mine + a.off_w) + row * a.k;
    T* dst = reinterpret_cast<T*>((char*)a.peer[s] + a.off_comb) + ((int64_t)a.rank * a.cap + slot) * a.H;
    for (int i = threadIdx.x; i < a.H / V; i += blockDim.x) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int q = 0; q < a.k; ++q) {
        int pos = pos_of_pair[row * a.k + q];
        if (pos < 0) continue;
        float wt = w[q];
        Vec16<T> v = ld_vec(y_sorted + (int64_t)pos * a.H + i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += wt * to_f(v.v[j]);
      }
      Vec16<T> o;
#pragma unroll
      for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(acc[j]);
      st_vec(dst + i * V, o);
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket + 1, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < a.R) {
    uint32_t* flag = reinterpret_cast<uint32_t*>((char*)a.peer[threadIdx.x] + a.off_comb_flag) + a.rank;
    st_release_u32(flag, epoch);
  }
  if (threadIdx.x == 0) a.ticket[1] = 0;
}

// One CTA per local token.
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_recv_kernel(EpArgs a, T* __restrict__ out, const T* __restrict__ addend) {
  constexpr int V = Vec16<T>::N;
  __shared__ int s_slot[8];
  const uint32_t epoch = *a.epoch + 1;
  const int64_t t = blockIdx.x;
  const bool live = t < a.T;  // a rank without local tokens runs one CTA that only advances the epoch
  char* mine = (char*)a.peer[a.rank];
  if (threadIdx.x < a.R) {
    const int d = threadIdx.x;
    const int slot = live ? a.sent_slot[t * a.R + d] : -1;
    s_slot[d] = slot;
    if (slot >= 0) {
      const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + a.off_comb_flag) + d;
      bool ok = false;
      for (uint32_t i = 0; i < a.spin_limit; ++i) {
        if (ld_acquire_u32(flag) == epoch) { ok = true; break; }
        if (i > 32) __nanosleep(64);
      }
      if (!ok) { atomicCAS(a.status, 0, 430 + d); s_slot[d] = -1; }
    }
  }
  __syncthreads();
  const T* comb = reinterpret_cast<const T*>(mine + a.off_comb);
  for (int i = threadIdx.x; live && i < a.H / V; i += blockDim.x) {
    float acc[V];
    if (addend != nullptr) {
      Vec16<T> v = ld_vec(addend + t * a.H + i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = to_f(v.v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
    }
    for (int d = 0; d < a.R; ++d) {
      const int slot = s_slot[d];
      if (slot < 0) continue;
      Vec16<T> v = ld_vec(comb + ((int64_t)d * a.cap + slot) * a.H + i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_f(v.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(acc[j]);
    st_vec(out + t * a.H + i * V, o);
  }
  // the call is over on this rank once every CTA is done: advance the epoch.  A rank with no local tokens still
  // launches one CTA (T clamped by the host) so that the epoch moves.
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket + 2, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    // wait (bounded) for the flags of ranks this rank sent nothing to as well, so that no peer is still writing
    // into the combine buffer when the next call starts
    for (int d = 0; d < a.R; ++d) {
      const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + a.off_comb_flag) + d;
      bool ok = false;
      for (uint32_t i = 0; i < a.spin_limit; ++i) {
        if (ld_acquire_u32(flag) == epoch) { ok = true; break; }
        if (i > 32) __nanosleep(64);
      }
      if (!ok) atomicCAS(a.status, 0, 440 + d);
    }
    a.ticket[2] = 0;
    *a.epoch = epoch;
  }
}

// scale_t[g][pos] = recv_scale[row][g] for every (row, expert slot) pair that was placed
__global__ void ep_permute_scales_kernel(float* __restrict__ scale_t, int64_t s_stride, const float* __restrict__ recv_scale,
                                         const int* __restrict__ pos_of_pair, int64_t pairs, int k, int ngroups) {
  const int64_t pair = blockIdx.x;
  if (pair >= pairs) return;
  const int pos = pos_of_pair[pair];
  if (pos < 0) return;
  const int64_t row = pair / k;
  for (int g = threadIdx.x; g < ngroups; g += blockDim.x) scale_t[(int64_t)g * s_stride + pos] = recv_scale[row * ngroups + g];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_ep_dispatch(const EpArgs* a, cudaStream_t st) {
  if (a->R > 8 || a->k > 32 || a->row_bytes % 16 || a->H % 128 || a->E % a->R) return 3;
  int64_t T = a->T;
  int blocks = (int)((T + 7) / 8);
  if (blocks < 1) blocks = 1;
  if (blocks > 1184) blocks = 1184;
  ep_dispatch_send_kernel<<<blocks, 256, 0, st>>>(*a);
  ep_dispatch_wait_kernel<<<a->R, 256, 0, st>>>(*a);
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_ep_permute_scales(float* scale_t, int64_t s_stride, const float* recv_scale, const int* pos_of_pair,
                                      int64_t pairs, int k, int ngroups, cudaStream_t st) {
  if (pairs == 0) return 0;
  ep_permute_scales_kernel<<<(unsigned)pairs, 64, 0, st>>>(scale_t, s_stride, recv_scale, pos_of_pair, pairs, k, ngroups);
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_ep_combine(const EpArgs* a, const void* y_sorted, const int* pos_of_pair, void* out, const void* addend,
                               int dtype, cudaStream_t st) {
  const unsigned rows = (unsigned)(a->R * a->cap);
  const unsigned tl = (unsigned)(a->T > 0 ? a->T : 1);
  EpArgs b = *a;
  B200_DISPATCH_DTYPE(dtype, {
    if (a->H % Vec16<T>::N) return 3;
    ep_combine_send_kernel<T><<<rows, 256, 0, st>>>(b, (const T*)y_sorted, pos_of_pair);
    ep_combine_recv_kernel<T><<<tl, 256, 0, st>>>(b, (T*)out, (const T*)addend);
  });
  return cudaGetLastError() != cudaSuccess;
}
