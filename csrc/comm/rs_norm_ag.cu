// Second half of the tensor-parallel "GEMM -> reduce-scatter -> add + RMSNorm -> all-gather -> GEMM"
// chain over NVLink peer memory (the first and last parts live in the GEMM kernel's epilogue /
// TMA producer, csrc/gemm/gemm_bf16.cu).
//
// Every rank owns Tloc = T / R consecutive tokens.  The row-parallel GEMM of each rank has stored
// its partial rows for my tokens into my staging area [src][local token][H] and bumped
// rs_flags[src][token tile] once per finished 128-feature tile.  This kernel, one CTA per few rows:
//   1. waits (bounded) until all R sources have delivered all H/128 tiles of the rows' token tile,
//   2. sums the R partials in rank order in fp32, adds the residual row and stores it back
//      (each rank maintains only its own rows of the residual),
//   3. RMS-normalises the row and stores it into the xfull buffer of EVERY rank (16-byte peer stores),
//   4. bumps ag_flags[token tile] on every rank by the number of rows delivered.
// The column-parallel GEMM that follows waits per token tile on those counters before its TMA loads.
// Counters of the previous call parity are re-zeroed here by CTA 0 (they are not in use any more:
// see the ordering argument in vllm_kunlun_b200/parallel/symm_mem.py).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

constexpr int kRnThreads = 512;

__device__ __forceinline__ uint32_t rn_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 rn_ld_relaxed_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void rn_red_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct RsNormParams {
  const void* stage;        // local [R][Tloc][H]
  const uint32_t* rs_flags; // local [R][max_tt] for this parity
  void* xfull[8];           // every rank's xfull [T][H]
  uint32_t* ag_flags[8];    // every rank's ag_flags [max_tt] for this parity
  uint32_t* reset_a; uint32_t* reset_b;
  int reset_a_n, reset_b_n;
  void* residual;           // full [T][H] tensor or null
  const void* weight;       // [H]
  int* status;
  int rank, R, Tloc, H, rs_bn, n_tiles, ag_bn, rows_per_cta, max_tt, gemma;
  float eps;
  uint32_t spin_limit;
};

template <typename T>
__global__ void __launch_bounds__(kRnThreads) rs_norm_ag_kernel(RsNormParams p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x;
  if (blockIdx.x == 0) {
    for (int i = tid; i < p.reset_a_n; i += kRnThreads) p.reset_a[i] = 0;
    for (int i = tid; i < p.reset_b_n; i += kRnThreads) p.reset_b[i] = 0;
  }
  const int tl0 = blockIdx.x * p.rows_per_cta;
  if (tl0 >= p.Tloc) return;
  const int tt_rs = tl0 / p.rs_bn;
  if (tid < p.R) {
    const uint32_t* f = p.rs_flags + tid * p.max_tt + tt_rs;
    bool ok = false;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
      if (rn_ld_acquire(f) >= (uint32_t)p.n_tiles) { ok = true; break; }
      if (i > 32) __nanosleep(64);
    }
    if (!ok) atomicCAS(p.status, 0, 300 + tid);
  }
  __syncthreads();
  const int nvec = p.H / V;
  const int rows = min(p.rows_per_cta, p.Tloc - tl0);
  for (int r = 0; r < rows; ++r) {
    const int tl = tl0 + r;
    const int64_t t = (int64_t)p.rank * p.Tloc + tl;
    float ss = 0.f;
    constexpr int kKeep = 4;
    float keep[kKeep][V];
    int k = 0;
    for (int i = tid; i < nvec; i += kRnThreads, ++k) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int s = 0; s < p.R; ++s) {
        const T* src = reinterpret_cast<const T*>(p.stage) + ((int64_t)s * p.Tloc + tl) * p.H + i * V;
        uint4 raw = rn_ld_relaxed_v4(src);
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f(v[j]);
      }
      Vec16<T> sum;
      if (p.residual != nullptr) {
        T* rr = reinterpret_cast<T*>(p.residual) + t * p.H + i * V;
        Vec16<T> res = ld_vec(rr);
#pragma unroll
        for (int j = 0; j < V; ++j) sum.v[j] = from_f<T>(to_f(from_f<T>(acc[j])) + to_f(res.v[j]));
        st_vec(rr, sum);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) sum.v[j] = from_f<T>(acc[j]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float f = to_f(sum.v[j]);
        ss += f * f;
        if (k < kKeep) keep[k][j] = f;
      }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / p.H + p.eps);
    k = 0;
    for (int i = tid; i < nvec; i += kRnThreads, ++k) {
      Vec16<T> w = ld_vec(reinterpret_cast<const T*>(p.weight) + i * V);
      Vec16<T> o;
      if (k < kKeep) {
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(keep[k][j] * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
      } else {
        Vec16<T> sv = ld_vec(reinterpret_cast<const T*>(p.residual) + t * p.H + i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(to_f(sv.v[j]) * inv * (to_f(w.v[j]) + (p.gemma ? 1.f : 0.f)));
      }
      for (int q = 0; q < p.R; ++q) st_vec(reinterpret_cast<T*>(p.xfull[q]) + t * p.H + i * V, o);
    }
    __syncthreads();
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.R) {
    const int64_t t0 = (int64_t)p.rank * p.Tloc + tl0;
    rn_red_add(p.ag_flags[tid] + t0 / p.ag_bn, (uint32_t)rows);
  }
}

// Blocks the stream until every token tile's arrival counter is complete (for consumers of the
// gathered activations that are not the fused GEMM).
__global__ void sp_wait_kernel(const uint32_t* flags, int n_tt, uint32_t expect, uint32_t spin_limit, int* status) {
  griddep_launch();
  griddep_wait();
  for (int tt = threadIdx.x; tt < n_tt; tt += blockDim.x) {
    bool ok = false;
    for (uint32_t i = 0; i < spin_limit; ++i) {
      if (rn_ld_acquire(flags + tt) >= expect) { ok = true; break; }
      if (i > 32) __nanosleep(64);
    }
    if (!ok) atomicCAS(status, 0, 400);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rs_norm_ag(const RsNormArgs* a, cudaStream_t st) {
  RsNormParams p;
  p.stage = a->stage; p.rs_flags = (const uint32_t*)a->rs_flags;
  for (int i = 0; i < 8; ++i) { p.xfull[i] = a->xfull[i]; p.ag_flags[i] = (uint32_t*)a->ag_flags[i]; }
  p.reset_a = (uint32_t*)a->reset_a; p.reset_b = (uint32_t*)a->reset_b; p.reset_a_n = a->reset_a_n; p.reset_b_n = a->reset_b_n;
  p.residual = a->residual; p.weight = a->weight; p.status = a->status;
  p.rank = a->rank; p.R = a->R; p.Tloc = a->Tloc; p.H = a->H; p.rs_bn = a->rs_bn; p.n_tiles = a->n_tiles;
  p.ag_bn = a->ag_bn; p.rows_per_cta = a->rows_per_cta; p.max_tt = a->max_tt; p.gemma = a->gemma; p.eps = a->eps;
  p.spin_limit = a->spin_limit;
  if (a->R > 8 || a->H % 8 || a->rows_per_cta < 1 || a->rs_bn % a->rows_per_cta || a->ag_bn % a->rows_per_cta) return 2;
  int grid = (a->Tloc + a->rows_per_cta - 1) / a->rows_per_cta;
  if (grid < 1) grid = 1;
  if (a->dtype == kBF16) return (int)launch_pdl(rs_norm_ag_kernel<__nv_bfloat16>, dim3(grid), dim3(kRnThreads), 0, st, p);
  if (a->dtype == kF16) return (int)launch_pdl(rs_norm_ag_kernel<__half>, dim3(grid), dim3(kRnThreads), 0, st, p);
  return 1;
}

extern "C" int b200_sp_wait(const void* flags, int n_tt, unsigned expect, unsigned spin_limit, int* status,
                            cudaStream_t st) {
  return (int)launch_pdl(sp_wait_kernel, dim3(1), dim3(128), 0, st, (const uint32_t*)flags, n_tt, (uint32_t)expect,
                         (uint32_t)spin_limit, status);
}
