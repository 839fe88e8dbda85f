// One-shot all-reduce over NVLink peer memory, optionally fused with residual add + RMSNorm.
//
// Every rank owns a symmetric buffer (same layout on all ranks, mapped into every peer):
//     [ data parity 0 | data parity 1 | flags[kMaxRanks][kMaxCtas] ]
// CTA c of every rank handles the same rows c, c + G, ...:
//   1. copy its rows of the local input into this rank's data[parity]          (local stores)
//   2. publish  flags(peer)[my_rank][c] = epoch  on every peer                 (st.release.sys)
//   3. wait until flags(me)[p][c] == epoch for every peer p                     (ld.acquire.sys, bounded)
//   4. read the rows from all ranks' data[parity] (plain peer loads), sum in rank order in fp32 -
//      every rank adds in the same order, so all ranks hold bit-identical results -
//      then either store, or add the residual, store it back and RMS-normalise the row.
// Two data parities make one barrier per call enough: a rank can only reach call k+2 (which
// reuses parity k) after every peer has entered call k+1, i.e. finished reading call k.
// The epoch is ONE call counter per communicator, kept in device memory (epochs[0]) and advanced by
// the kernel itself (the last CTA to finish, found through the ticket in epochs[1]), so CUDA-graph
// replays need no host-side reset and every CTA of a call - whatever the grid or the row width of
// this and earlier calls - works with the same epoch and the same parity.  The wait is bounded; on
// time-out the status word is set and the kernel completes (with wrong data) instead of hanging
// the GPU; the host reads the word with every step's result.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

constexpr int kArMaxRanks = 8;
constexpr int kArMaxCtas = 128;
constexpr int kArThreads = 512;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

struct ArParams {
  void* bufs[kArMaxRanks];   // symmetric buffers of all ranks, as mapped in this process
  const void* in;            // [rows, H] local partial sums
  void* out;                 // [rows, H]
  void* residual;            // [rows, H] (fused norm) or null
  const void* weight;        // [H] (fused norm) or null
  uint32_t* epochs;          // [0] completed calls of this communicator, [1] finished-CTA ticket of the running call
  int* status;
  int64_t parity_bytes;      // size of one data parity
  int64_t flags_offset;      // byte offset of the flag block inside a symmetric buffer
  int rank, nranks, rows, H;
  float eps;
  int gemma;
  uint32_t spin_limit;
  int64_t ll_slot_bytes;     // low-latency variant: bytes of one (parity, source) slot of a symmetric buffer
  int skip_push;             // low-latency variant: the producer of `in` (a GEMM epilogue) has already pushed it
};

// Called by every CTA after its last use of the epoch: the last one publishes the finished call.
__device__ __forceinline__ void finish_call(uint32_t* epochs, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&epochs[1], 1u);
    if (t == gridDim.x - 1) {
      epochs[1] = 0;
      __threadfence();
      epochs[0] = epoch;
    }
  }
}

template <typename T, bool kNorm>
__global__ void __launch_bounds__(kArThreads) oneshot_allreduce_kernel(ArParams p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int c = blockIdx.x, G = gridDim.x;
  const int tid = threadIdx.x;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.epochs) + 1;
  const int parity = epoch & 1;
  const int nvec = p.H / V;
  T* my_data = reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(p.bufs[p.rank]) + parity * p.parity_bytes);

  // 1. stage my partial rows
  for (int row = c; row < p.rows; row += G) {
    const T* src = reinterpret_cast<const T*>(p.in) + (int64_t)row * p.H;
    T* dst = my_data + (int64_t)row * p.H;
    for (int i = tid; i < nvec; i += kArThreads) st_vec(dst + i * V, ld_vec(src + i * V));
  }
  __threadfence_system();
  __syncthreads();
  // 2./3. signal every peer, then wait for every peer
  if (tid < p.nranks) {
    uint32_t* peer_flags = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.bufs[tid]) + p.flags_offset);
    st_release_sys(peer_flags + p.rank * kArMaxCtas + c, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(reinterpret_cast<uint8_t*>(p.bufs[p.rank]) + p.flags_offset) +
                           tid * kArMaxCtas + c;
    bool ok = false;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
      if (i > 64) __nanosleep(64);
    }
    if (!ok) atomicCAS(p.status, 0, 200 + tid);
  }
  __syncthreads();

  // 4. reduce (and normalise)
  for (int row = c; row < p.rows; row += G) {
    float ss = 0.f;
    // each thread owns the vectors tid, tid + 512, ... of the row; H <= 512 * V * kMaxKeep keeps them in registers
    constexpr int kMaxKeep = 4;
    float keep[kMaxKeep][V];
    int k = 0;
    for (int i = tid; i < nvec; i += kArThreads, ++k) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int r = 0; r < p.nranks; ++r) {
        const T* src = reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(p.bufs[r]) + parity * p.parity_bytes) +
                       (int64_t)row * p.H + i * V;
        uint4 raw = ld_relaxed_sys_v4(src);
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f(v[j]);
      }
      if (kNorm) {
        T* rr = reinterpret_cast<T*>(p.residual) + (int64_t)row * p.H + i * V;
        Vec16<T> res = ld_vec(rr);
        Vec16<T> sum;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          // round the all-reduced value to T first (what a separate all-reduce would hand to add+norm)
          float s = to_f(from_f<T>(acc[j])) + to_f(res.v[j]);
          sum.v[j] = from_f<T>(s);
          float f = to_f(sum.v[j]);
          ss += f * f;
          if (k < kMaxKeep) keep[k][j] = f;
        }
        st_vec(rr, sum);
      } else {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(acc[j]);
        st_vec(reinterpret_cast<T*>(p.out) + (int64_t)row * p.H + i * V, o);
      }
    }
    if (kNorm) {
      ss = block_sum(ss, red);
      const float inv = rsqrtf(ss / p.H + p.eps);
      k = 0;
      for (int i = tid; i < nvec; i += kArThreads, ++k) {
        Vec16<T> w = ld_vec(reinterpret_cast<const T*>(p.weight) + i * V);
        Vec16<T> o;
        if (k < kMaxKeep) {
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(keep[k][j] * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
        } else {
          Vec16<T> s = ld_vec(reinterpret_cast<const T*>(p.residual) + (int64_t)row * p.H + i * V);
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(to_f(s.v[j]) * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
        }
        st_vec(reinterpret_cast<T*>(p.out) + (int64_t)row * p.H + i * V, o);
      }
      __syncthreads();
    }
  }
  finish_call(p.epochs, epoch);
}


// ---- low-latency variant for decode-sized payloads -------------------------------------------------------------
// Every 4 bytes of payload travel in an 8-byte unit {data, epoch}, written straight into the DESTINATION rank's
// buffer (slot [parity][source]) with 16-byte stores whose 8-byte halves are each written atomically.  A receiver
// polls its own memory until all units of a vector carry the current epoch: arrival of the flag is arrival of the
// data, so no fence, no separate flag store and no remote load is on the critical path - one NVLink traversal
// instead of three.  Sums are taken in rank order (own contribution from the input tensor), so all ranks end up
// with the same bits.  Two parities for the same reason as above; epochs live in device memory.
__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename T, bool kNorm>
__global__ void __launch_bounds__(kArThreads) ll_allreduce_kernel(ArParams p) {
  static_assert(sizeof(T) == 2, "16-bit payloads");
  constexpr int V = 8;
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int c = blockIdx.x, G = gridDim.x, tid = threadIdx.x;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.epochs) + 1;
  const int parity = epoch & 1;
  const int nvec = p.H / V;
  const int64_t row_bytes = (int64_t)p.H * 4;  // 2 H bytes of payload, doubled by the flags
  auto slot = [&](int dest, int src) {
    return reinterpret_cast<uint8_t*>(p.bufs[dest]) + ((int64_t)parity * p.nranks + src) * p.ll_slot_bytes;
  };
  // 1. push my rows to every peer (unless the kernel that produced them already has)
  for (int row = c; row < p.rows && !p.skip_push; row += G) {
    for (int i = tid; i < nvec; i += kArThreads) {
      const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.in) + (int64_t)row * p.H + i * V);
      for (int d = 0; d < p.nranks; ++d) {
        if (d == p.rank) continue;
        uint8_t* dst = slot(d, p.rank) + row * row_bytes + (int64_t)i * 32;
        st_volatile_v4(dst, v.x, epoch, v.y, epoch);
        st_volatile_v4(dst + 16, v.z, epoch, v.w, epoch);
      }
    }
  }
  // 2. collect and reduce
  for (int row = c; row < p.rows; row += G) {
    float ss = 0.f;
    constexpr int kMaxKeep = 4;
    float keep[kMaxKeep][V];
    int k = 0;
    for (int i = tid; i < nvec; i += kArThreads, ++k) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int r = 0; r < p.nranks; ++r) {
        uint4 raw;
        if (r == p.rank) {
          raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.in) + (int64_t)row * p.H + i * V);
        } else {
          const uint8_t* src = slot(p.rank, r) + row * row_bytes + (int64_t)i * 32;
          bool ok = false;
          for (uint32_t it = 0; it < p.spin_limit; ++it) {
            uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(src + 16);
            if (a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch) {
              raw = make_uint4(a.x, a.z, b.x, b.z);
              ok = true;
              break;
            }
            if (it > 4096) __nanosleep(32);
          }
          if (!ok) { atomicCAS(p.status, 0, 210 + r); raw = make_uint4(0, 0, 0, 0); }
        }
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f(v[j]);
      }
      if (kNorm) {
        T* rr = reinterpret_cast<T*>(p.residual) + (int64_t)row * p.H + i * V;
        Vec16<T> res = ld_vec(rr);
        Vec16<T> sum;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float s = to_f(from_f<T>(acc[j])) + to_f(res.v[j]);
          sum.v[j] = from_f<T>(s);
          float f = to_f(sum.v[j]);
          ss += f * f;
          if (k < kMaxKeep) keep[k][j] = f;
        }
        st_vec(rr, sum);
      } else {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(acc[j]);
        st_vec(reinterpret_cast<T*>(p.out) + (int64_t)row * p.H + i * V, o);
      }
    }
    if (kNorm) {
      ss = block_sum(ss, red);
      const float inv = rsqrtf(ss / p.H + p.eps);
      k = 0;
      for (int i = tid; i < nvec; i += kArThreads, ++k) {
        Vec16<T> w = ld_vec(reinterpret_cast<const T*>(p.weight) + i * V);
        Vec16<T> o;
        if (k < kMaxKeep) {
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(keep[k][j] * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
        } else {
          Vec16<T> s2 = ld_vec(reinterpret_cast<const T*>(p.residual) + (int64_t)row * p.H + i * V);
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(to_f(s2.v[j]) * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
        }
        st_vec(reinterpret_cast<T*>(p.out) + (int64_t)row * p.H + i * V, o);
      }
      __syncthreads();
    }
  }
  finish_call(p.epochs, epoch);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_allreduce_max_ctas() { return kArMaxCtas; }
extern "C" int64_t b200_allreduce_flag_bytes() { return (int64_t)kArMaxRanks * kArMaxCtas * sizeof(uint32_t); }

extern "C" int b200_oneshot_allreduce(void* const* bufs, const void* in, void* out, void* residual, const void* weight,
                                      uint32_t* epochs, int* status, int64_t parity_bytes, int64_t flags_offset,
                                      int rank, int nranks, int rows, int H, float eps, int gemma, int grid,
                                      uint32_t spin_limit, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (nranks > kArMaxRanks || grid > kArMaxCtas || grid < 1) return 2;
  ArParams p;
  for (int i = 0; i < kArMaxRanks; ++i) p.bufs[i] = i < nranks ? bufs[i] : nullptr;
  p.in = in; p.out = out; p.residual = residual; p.weight = weight; p.epochs = epochs; p.status = status;
  p.parity_bytes = parity_bytes; p.flags_offset = flags_offset; p.rank = rank; p.nranks = nranks; p.rows = rows;
  p.H = H; p.eps = eps; p.gemma = gemma; p.spin_limit = spin_limit; p.ll_slot_bytes = 0; p.skip_push = 0;
  if (dtype == kBF16) {
    if (H % 8) return 2;
    if (residual) launch_pdl(oneshot_allreduce_kernel<__nv_bfloat16, true>, dim3(grid), dim3(kArThreads), 0, st, p);
    else launch_pdl(oneshot_allreduce_kernel<__nv_bfloat16, false>, dim3(grid), dim3(kArThreads), 0, st, p);
  } else if (dtype == kF16) {
    if (H % 8) return 2;
    if (residual) launch_pdl(oneshot_allreduce_kernel<__half, true>, dim3(grid), dim3(kArThreads), 0, st, p);
    else launch_pdl(oneshot_allreduce_kernel<__half, false>, dim3(grid), dim3(kArThreads), 0, st, p);
  } else if (dtype == kF32) {
    if (H % 4) return 2;
    if (residual) launch_pdl(oneshot_allreduce_kernel<float, true>, dim3(grid), dim3(kArThreads), 0, st, p);
    else launch_pdl(oneshot_allreduce_kernel<float, false>, dim3(grid), dim3(kArThreads), 0, st, p);
  } else {
    return 1;
  }
  return (int)cudaGetLastError();
}

// Low-latency all-reduce (see ll_allreduce_kernel): `bufs` are the ranks' LL buffers of 2 * nranks slots each.
extern "C" int b200_ll_allreduce(void* const* bufs, const void* in, void* out, void* residual, const void* weight,
                                 uint32_t* epochs, int* status, int64_t slot_bytes, int rank, int nranks, int rows, int H,
                                 float eps, int gemma, int grid, uint32_t spin_limit, int skip_push, int dtype,
                                 cudaStream_t st) {
  if (rows == 0) return 0;
  if (nranks > kArMaxRanks || grid > kArMaxCtas || grid < 1 || H % 8 || (int64_t)rows * H * 4 > slot_bytes) return 2;
  ArParams p;
  for (int i = 0; i < kArMaxRanks; ++i) p.bufs[i] = i < nranks ? bufs[i] : nullptr;
  p.in = in; p.out = out; p.residual = residual; p.weight = weight; p.epochs = epochs; p.status = status;
  p.parity_bytes = 0; p.flags_offset = 0; p.rank = rank; p.nranks = nranks; p.rows = rows;
  p.H = H; p.eps = eps; p.gemma = gemma; p.spin_limit = spin_limit; p.ll_slot_bytes = slot_bytes;
  p.skip_push = skip_push;
  if (dtype == kBF16) {
    if (residual) launch_pdl(ll_allreduce_kernel<__nv_bfloat16, true>, dim3(grid), dim3(kArThreads), 0, st, p);
    else launch_pdl(ll_allreduce_kernel<__nv_bfloat16, false>, dim3(grid), dim3(kArThreads), 0, st, p);
  } else if (dtype == kF16) {
    if (residual) launch_pdl(ll_allreduce_kernel<__half, true>, dim3(grid), dim3(kArThreads), 0, st, p);
    else launch_pdl(ll_allreduce_kernel<__half, false>, dim3(grid), dim3(kArThreads), 0, st, p);
  } else {
    return 1;
  }
  return (int)cudaGetLastError();
}
