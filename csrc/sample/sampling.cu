// Vocabulary-wide sampling kernels: temperature + top-k + top-p + exponential-race draw in one launch,
// repetition penalty, and the speculative-decoding rejection sampler.
//
// Behaviour matches the sort-based masking of the reference's TopKTopPSampler
// (vllm_kunlun/v1/sample/ops/topk_topp_sampler.py:51-216): keep logits >= the k-th largest, then drop the
// low-probability tail whose cumulative mass is <= 1 - p, then draw argmax(prob / Exp(1)) (:141-174).
// Instead of sorting the row, both thresholds come from an MSB-first radix select over the float bit
// patterns (count histogram for top-k, probability-mass histogram for top-p): 4 passes of 8 bits each.
#include <cooperative_groups.h>

#include "../api.h"
#include "../common/utils.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_bits(float v) {  // monotone float -> uint32
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unorder_bits(uint32_t u) {
  uint32_t b = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
  return __uint_as_float(b);
}
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
// Exp(1) variate from a counter-based hash of (seed, row, column)
__device__ __forceinline__ float exp_variate(uint64_t seed, uint64_t row, uint64_t col) {
  uint64_t h = mix64(seed ^ mix64(row * 0x100000001b3ull + col));
  float u = ((h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(u);
}

template <typename T>
__device__ __forceinline__ float scaled(const T* row, int i, float inv_t) { return to_f(row[i]) * inv_t; }

struct ArgBest { float v; int i; };
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ ArgBest block_argbest(ArgBest x, ArgBest* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y{__shfl_xor_sync(0xffffffff, x.v, o), __shfl_xor_sync(0xffffffff, x.i, o)};
    x = better(x, y);
  }
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = x;
  __syncthreads();
  ArgBest r = (l < nw) ? red[l] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y{__shfl_xor_sync(0xffffffff, r.v, o), __shfl_xor_sync(0xffffffff, r.i, o)};
    r = better(r, y);
  }
  return r;
}

// One block per row.
template <typename T>
__global__ void __launch_bounds__(kThreads) topk_topp_sample_kernel(
    int64_t* __restrict__ out, const T* __restrict__ logits, int64_t stride, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ noise, int64_t noise_stride,
    uint64_t seed, uint64_t step) {
  __shared__ float red[32];
  __shared__ ArgBest ared[32];
  __shared__ float hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ float s_below;
  __shared__ int s_need;
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + row * stride;
  const float temp = temperature ? temperature[row] : 1.f;

  if (temp == 0.f) {  // greedy: smallest index among the maxima
    ArgBest b{-INFINITY, 0x7fffffff};
    for (int i = tid; i < V; i += kThreads) b = better(b, ArgBest{to_f(x[i]), i});
    b = block_argbest(b, ared);
    if (tid == 0) out[row] = b.i;
    return;
  }
  const float inv_t = 1.f / temp;
  int k = top_k ? top_k[row] : 0;
  if (k <= 0 || k > V) k = V;
  const float p = top_p ? top_p[row] : 1.f;

  float m = -INFINITY;
  for (int i = tid; i < V; i += kThreads) m = fmaxf(m, scaled(x, i, inv_t));
  m = block_max(m, red);

  // ---- top-k threshold: k-th largest scaled logit (ties kept), by counting radix select
  float thr_k = -INFINITY;
  if (k < V) {
    uint32_t prefix = 0;
    int need = k;  // rank from the top within the current prefix bucket
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      if (tid < 256) hist[tid] = 0.f;
      __syncthreads();
      for (int i = tid; i < V; i += kThreads) {
        uint32_t u = order_bits(scaled(x, i, inv_t));
        if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1.f);
      }
      __syncthreads();
      if (tid == 0) {
        int acc = 0, d = 255;
        for (; d > 0; --d) {
          int c = (int)hist[d];
          if (acc + c >= need) break;
          acc += c;
        }
        s_prefix = prefix | ((uint32_t)d << shift);
        s_need = need - acc;
      }
      __syncthreads();
      prefix = s_prefix;
      need = s_need;
    }
    thr_k = unorder_bits(prefix);
  }

  // ---- soft-max denominator over the top-k survivors
  float z = 0.f;
  for (int i = tid; i < V; i += kThreads) {
    float l = scaled(x, i, inv_t);
    if (l >= thr_k) z += __expf(l - m);
  }
  z = block_sum(z, red);

  // ---- top-p threshold on e = exp(l - m): drop the ascending tail whose mass is <= (1 - p) * z
  float thr_p = 0.f;
  if (p < 1.f) {
    const float budget = (1.f - p) * z;
    uint32_t prefix = 0;
    float below = 0.f;  // mass of everything strictly under the current prefix bucket
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      if (tid < 256) hist[tid] = 0.f;
      __syncthreads();
      for (int i = tid; i < V; i += kThreads) {
        float l = scaled(x, i, inv_t);
        if (l < thr_k) continue;
        float e = __expf(l - m);
        uint32_t u = __float_as_uint(e);  // e >= 0: the bit pattern is already monotone
        if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], e);
      }
      __syncthreads();
      if (tid == 0) {
        float acc = below, acc_last = below;
        int d = 0, last = -1;
        for (; d < 256; ++d) {
          if (hist[d] > 0.f) { last = d; acc_last = acc; }
          if (acc + hist[d] > budget) break;
          acc += hist[d];
        }
        if (d == 256) {  // rounding left the budget unreached: keep the highest occupied bucket
          d = last < 0 ? 0 : last;
          acc = acc_last;
        }
        s_prefix = prefix | ((uint32_t)d << shift);
        s_below = acc;
      }
      __syncthreads();
      prefix = s_prefix;
      below = s_below;
    }
    thr_p = __uint_as_float(prefix);
  }

  // ---- exponential race over the survivors
  ArgBest b{-INFINITY, 0x7fffffff};
  for (int i = tid; i < V; i += kThreads) {
    float l = scaled(x, i, inv_t);
    if (l < thr_k) continue;
    float e = __expf(l - m);
    if (e < thr_p) continue;
    float q = noise ? noise[row * noise_stride + i] : exp_variate(seed, step * 65536ull + row, i);
    b = better(b, ArgBest{e / q, i});
  }
  b = block_argbest(b, ared);
  if (tid == 0) out[row] = b.i;
}

// ---- cluster version: 8 CTAs share a row, every thread keeps its elements in registers ------------------------
// All passes after the load run out of registers.  Thresholds are found by refining a value interval: each pass
// splits the current interval of scaled logits into 256 equal bins (spread-out bins keep shared-memory atomics
// from piling onto one address, unlike digit histograms of float bit patterns, whose leading digits are almost
// constant), the 8 CTAs' histograms are summed through distributed shared memory, and the bin that contains the
// k-th largest element (top-k, by count) or the point where the low-probability tail reaches 1 - p (top-p, by
// mass) becomes the next interval.  Four passes narrow the interval to range * 2^-32, i.e. to ties.
// Used whenever the row fits (V <= 8 * 1024 * kMaxPerThread).
constexpr int kCluster = 8;
constexpr int kMaxPerThread = 24;
constexpr int kRefine = 4;

struct ClusterScratch {
  float hist[2][256];
  float val[4];
  ArgBest best;
};

__device__ __forceinline__ float cluster_reduce(cg::cluster_group& cl, ClusterScratch* s, float v, float* red, int slot,
                                                int op /*0 sum, 1 max, 2 min*/) {
  v = op == 0 ? block_sum(v, red) : (op == 1 ? block_max(v, red) : -block_max(-v, red));
  if (threadIdx.x == 0) s->val[slot] = v;
  cl.sync();
  float acc = op == 0 ? 0.f : (op == 1 ? -INFINITY : INFINITY);
  for (int r = 0; r < kCluster; ++r) {
    float o = cl.map_shared_rank(s, r)->val[slot];
    acc = op == 0 ? acc + o : (op == 1 ? fmaxf(acc, o) : fminf(acc, o));
  }
  return acc;
}

template <typename T, int NPT>
__global__ void __cluster_dims__(kCluster, 1, 1) __launch_bounds__(kThreads) topk_topp_sample_cluster_kernel(
    int64_t* __restrict__ out, const T* __restrict__ logits, int64_t stride, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ noise, int64_t noise_stride,
    uint64_t seed, uint64_t step) {
  __shared__ ClusterScratch sc;
  __shared__ float red[32];
  __shared__ float s_tot[256];  // cluster-wide histogram totals (identical in every CTA)
  __shared__ ArgBest ared[32];
  __shared__ int s_bin;
  __shared__ float s_acc;
  cg::cluster_group cl = cg::this_cluster();
  const int crank = (int)cl.block_rank();
  const int row = blockIdx.x / kCluster, tid = threadIdx.x;
  const T* x = logits + row * stride;
  const float temp = temperature ? temperature[row] : 1.f;
  const bool greedy = temp == 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  // element j of this thread: interleaved over the cluster so that every load instruction is coalesced
  float l[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    const int i = (j * kCluster + crank) * kThreads + tid;
    l[j] = i < V ? to_f(x[i]) * inv_t : -INFINITY;
  }
  auto index_of = [&](int j) { return (j * kCluster + crank) * kThreads + tid; };
  auto cluster_argbest = [&](ArgBest bb) {
    bb = block_argbest(bb, ared);
    if (tid == 0) sc.best = bb;
    cl.sync();
    ArgBest r{-INFINITY, 0x7fffffff};
    for (int c = 0; c < kCluster; ++c) r = better(r, cl.map_shared_rank(&sc, c)->best);
    return r;
  };

  if (greedy) {
    ArgBest bb{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int j = 0; j < NPT; ++j) bb = better(bb, ArgBest{l[j], index_of(j)});
    bb = cluster_argbest(bb);
    if (crank == 0 && tid == 0) out[row] = bb.i;
    cl.sync();  // nobody leaves while its shared memory may still be read
    return;
  }
  int k = top_k ? top_k[row] : 0;
  if (k <= 0 || k > V) k = V;
  const float p = top_p ? top_p[row] : 1.f;

  float m = -INFINITY, lowest = INFINITY;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    m = fmaxf(m, l[j]);
    if (l[j] != -INFINITY) lowest = fminf(lowest, l[j]);
  }
  m = cluster_reduce(cl, &sc, m, red, 0, 1);
  lowest = cluster_reduce(cl, &sc, lowest, red, 1, 2);

  // element state: bit j of `keep` = survives, bit j of `alive` = inside the interval still being refined
  uint32_t keep = 0, alive = 0;
#pragma unroll
  for (int j = 0; j < NPT; ++j)
    if (l[j] != -INFINITY) alive |= 1u << j;
  int pass_no = 0;  // selects the histogram buffer: a buffer is rewritten two cluster syncs after its last read

  // One refinement pass.  `by_mass`: histogram of exp(l - m) walked from the bottom until `target` is exceeded
  // (elements under the chosen bin are dropped); otherwise a count histogram walked from the top until `target`
  // elements are covered (elements above the chosen bin are kept).  Returns the chosen bin's interval in lo / hi
  // and the amount accumulated outside it in `acc`.
  auto refine = [&](bool by_mass, float& lo, float& hi, float target, float& acc_out) {
    float* h = sc.hist[pass_no & 1];
    for (int i = tid; i < 256; i += kThreads) h[i] = 0.f;
    __syncthreads();
    const float scale = 256.f / fmaxf(hi - lo, 1e-30f);
    int bins[NPT];
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      bins[j] = -1;
      if (!(alive >> j & 1)) continue;
      int bi = (int)((l[j] - lo) * scale);
      bi = bi < 0 ? 0 : (bi > 255 ? 255 : bi);
      bins[j] = bi;
      atomicAdd(&h[bi], by_mass ? __expf(l[j] - m) : 1.f);
    }
    cl.sync();
    if (tid < 256) {
      float c = 0.f;
      for (int r = 0; r < kCluster; ++r) c += cl.map_shared_rank(&sc, r)->hist[pass_no & 1][tid];  // fixed order
      s_tot[tid] = c;
    }
    __syncthreads();
    if (tid == 0) {
      float acc = acc_out;
      int d;
      if (by_mass) {
        int last = -1;
        float acc_last = acc;
        for (d = 0; d < 256; ++d) {
          if (s_tot[d] > 0.f) { last = d; acc_last = acc; }
          if (acc + s_tot[d] > target) break;
          acc += s_tot[d];
        }
        if (d == 256) { d = last < 0 ? 0 : last; acc = acc_last; }  // rounding: stay on the highest occupied bin
      } else {
        for (d = 255; d > 0; --d) {
          if (acc + s_tot[d] >= target) break;
          acc += s_tot[d];
        }
      }
      s_bin = d;
      s_acc = acc;
    }
    __syncthreads();
    const int d = s_bin;
    acc_out = s_acc;
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      if (bins[j] < 0 || bins[j] == d) continue;
      alive &= ~(1u << j);
      if (bins[j] > d) keep |= 1u << j;  // above the boundary bin: kept by both criteria
    }
    const float width = (hi - lo) * (1.f / 256.f);
    lo = lo + width * d;
    hi = lo + width;
    ++pass_no;
  };

  // ---- top-k: count from the top
  if (k < V) {
    float lo = lowest, hi = m + fmaxf(fabsf(m), 1.f) * 1e-6f, covered = 0.f;
    for (int r = 0; r < kRefine; ++r) refine(false, lo, hi, (float)k, covered);
  }
  keep |= alive;  // whatever is still inside the last interval ties with the k-th element
  alive = keep;
  keep = 0;

  // ---- soft-max denominator over the survivors
  float z = 0.f;
  float low2 = INFINITY;
#pragma unroll
  for (int j = 0; j < NPT; ++j)
    if (alive >> j & 1) { z += __expf(l[j] - m); low2 = fminf(low2, l[j]); }
  z = cluster_reduce(cl, &sc, z, red, 2, 0);

  // ---- top-p: mass from the bottom
  if (p < 1.f) {
    low2 = cluster_reduce(cl, &sc, low2, red, 3, 2);
    float lo = low2, hi = m + fmaxf(fabsf(m), 1.f) * 1e-6f, below = 0.f;
    const float budget = (1.f - p) * z;
    for (int r = 0; r < kRefine; ++r) refine(true, lo, hi, budget, below);
  }
  keep |= alive;

  // ---- exponential race
  ArgBest bb{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    if (!(keep >> j & 1)) continue;
    const int i = index_of(j);
    float q = noise ? noise[row * noise_stride + i] : exp_variate(seed, step * 65536ull + row, i);
    bb = better(bb, ArgBest{__expf(l[j] - m) / q, i});
  }
  bb = cluster_argbest(bb);
  if (crank == 0 && tid == 0) out[row] = bb.i;
  cl.sync();
}

// logits[b, tok] /= or *= penalty once per distinct token of the row's history
template <typename T>
__global__ void repetition_penalty_kernel(T* __restrict__ logits, int64_t stride, int V, const int64_t* __restrict__ tokens,
                                          int64_t tok_stride, const int* __restrict__ n_tokens,
                                          const float* __restrict__ penalty, uint32_t* __restrict__ seen /*[B, ceil(V/32)]*/) {
  const int row = blockIdx.y;
  const float pen = penalty[row];
  if (pen == 1.f) return;
  const int n = n_tokens[row];
  const int words = (V + 31) / 32;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x) {
    int64_t t = tokens[row * tok_stride + j];
    if (t < 0 || t >= V) continue;
    uint32_t bit = 1u << (t & 31);
    uint32_t old = atomicOr(&seen[(int64_t)row * words + (t >> 5)], bit);
    if (old & bit) continue;
    float l = to_f(logits[row * stride + t]);
    logits[row * stride + t] = from_f<T>(l > 0.f ? l / pen : l * pen);
  }
}

// One block per request.  probs are fp32 [n, V] (flat over all draft positions).
__global__ void __launch_bounds__(kThreads) rejection_sample_kernel(
    int64_t* __restrict__ out /*[B, S+1]*/, int S, const int64_t* __restrict__ draft_ids, const int* __restrict__ cu_draft,
    const float* __restrict__ target_probs, const float* __restrict__ draft_probs, int V,
    const int64_t* __restrict__ bonus, const uint8_t* __restrict__ is_greedy, const float* __restrict__ uniform,
    const float* __restrict__ recover_q, uint64_t seed, uint64_t step) {
  __shared__ ArgBest ared[32];
  __shared__ int s_stop;
  const int b = blockIdx.x, tid = threadIdx.x;
  const int s0 = cu_draft[b], nd = cu_draft[b + 1] - s0;
  const bool greedy = is_greedy[b] != 0;
  for (int j = tid; j <= S; j += kThreads) out[(int64_t)b * (S + 1) + j] = -1;
  __syncthreads();
  int pos = 0;
  for (; pos < nd; ++pos) {
    const int64_t fl = s0 + pos;
    const int64_t d = draft_ids[fl];
    const float* tp = target_probs + fl * V;
    bool ok;
    if (greedy) {
      ArgBest a{-INFINITY, 0x7fffffff};
      for (int i = tid; i < V; i += kThreads) a = better(a, ArgBest{tp[i], i});
      a = block_argbest(a, ared);
      ok = a.i == d;
      if (!ok && tid == 0) out[(int64_t)b * (S + 1) + pos] = a.i;
    } else {
      float pt = tp[d], pd = draft_probs ? draft_probs[fl * V + d] : 1.f;
      float u = uniform ? uniform[fl] : ((mix64(seed ^ mix64(step * 1315423911ull + fl)) >> 40) + 0.5f) * (1.f / 16777216.f);
      ok = pd > 0.f && pt / fmaxf(pd, 1e-30f) >= u;
      if (!ok) {  // recovered distribution max(pt - pd, 0) (draft token zeroed when no draft probs)
        ArgBest a{-INFINITY, 0x7fffffff};
        for (int i = tid; i < V; i += kThreads) {
          float adj = draft_probs ? fmaxf(tp[i] - draft_probs[fl * V + i], 0.f) : (i == d ? 0.f : tp[i]);
          float q = recover_q ? recover_q[(int64_t)b * V + i] : exp_variate(seed ^ 0x5bd1e995ull, step * 65536ull + b, i);
          a = better(a, ArgBest{adj / q, i});
        }
        a = block_argbest(a, ared);
        if (tid == 0) out[(int64_t)b * (S + 1) + pos] = a.i;
      }
    }
    if (tid == 0) s_stop = ok ? 0 : 1;
    __syncthreads();
    if (s_stop) return;
    if (tid == 0) out[(int64_t)b * (S + 1) + pos] = d;
    __syncthreads();
  }
  if (tid == 0) out[(int64_t)b * (S + 1) + nd] = bonus[b];
}

}  // namespace
}  // namespace b200

extern "C" int b200_topk_topp_sample(int64_t* out, const void* logits, int64_t rows, int V, int64_t stride,
                                     const float* temperature, const int* top_k, const float* top_p, const float* noise,
                                     int64_t noise_stride, uint64_t seed, uint64_t step, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  const int per = (V + b200::kCluster * b200::kThreads - 1) / (b200::kCluster * b200::kThreads);
  if (per <= b200::kMaxPerThread) {
    const unsigned grid = (unsigned)rows * b200::kCluster;
#define B200_SAMPLE_CASE(NPT)                                                                                            \
  B200_DISPATCH_DTYPE(dtype, (b200::topk_topp_sample_cluster_kernel<T, NPT><<<grid, b200::kThreads, 0, st>>>(             \
                                 out, (const T*)logits, stride, V, temperature, top_k, top_p, noise, noise_stride, seed, step)))
    if (per <= 4) { B200_SAMPLE_CASE(4); }
    else if (per <= 8) { B200_SAMPLE_CASE(8); }
    else if (per <= 16) { B200_SAMPLE_CASE(16); }
    else { B200_SAMPLE_CASE(24); }
#undef B200_SAMPLE_CASE
    return cudaGetLastError() != cudaSuccess;
  }
  B200_DISPATCH_DTYPE(dtype, (b200::topk_topp_sample_kernel<T><<<(unsigned)rows, b200::kThreads, 0, st>>>(
                                 out, (const T*)logits, stride, V, temperature, top_k, top_p, noise, noise_stride, seed, step)));
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_repetition_penalty(void* logits, int64_t rows, int V, int64_t stride, const int64_t* tokens,
                                       int64_t tok_stride, int max_tokens, const int* n_tokens, const float* penalty,
                                       uint32_t* seen, int dtype, cudaStream_t st) {
  if (rows == 0 || max_tokens == 0) return 0;
  if (cudaMemsetAsync(seen, 0, (size_t)rows * ((V + 31) / 32) * 4, st) != cudaSuccess) return 2;
  dim3 grid((unsigned)((max_tokens + 255) / 256 > 64 ? 64 : (max_tokens + 255) / 256), (unsigned)rows);
  B200_DISPATCH_DTYPE(dtype, (b200::repetition_penalty_kernel<T><<<grid, 256, 0, st>>>(
                                 (T*)logits, stride, V, tokens, tok_stride, n_tokens, penalty, seen)));
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_rejection_sample(int64_t* out, int64_t B, int S, const int64_t* draft_ids, const int* cu_draft,
                                     const float* target_probs, const float* draft_probs, int V, const int64_t* bonus,
                                     const uint8_t* is_greedy, const float* uniform, const float* recover_q, uint64_t seed,
                                     uint64_t step, cudaStream_t st) {
  if (B == 0) return 0;
  b200::rejection_sample_kernel<<<(unsigned)B, b200::kThreads, 0, st>>>(out, S, draft_ids, cu_draft, target_probs, draft_probs,
                                                                        V, bonus, is_greedy, uniform, recover_q, seed, step);
  return cudaGetLastError() != cudaSuccess;
}
