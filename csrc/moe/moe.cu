// MoE routing, permutation and fp8 activation quantisation kernels.
//
// route:     one warp per token over E <= 512 experts: softmax / sigmoid(+bias, group-limited) /
//            top-k-then-softmax, k <= 16 rounds of warp arg-max (ties -> lowest expert id).
// permute:   histogram of (token, slot) pairs per local expert -> exclusive scan (lod) -> scatter of
//            token rows into expert-sorted order; pairs routed to non-local experts are dropped.
// unpermute: out[t] = sum_j w[t, j] * y_sorted[pos(t, j)]   (fixed j order: deterministic)
// quant:     dynamic 1x128 e4m3 quantisation, scales stored transposed [K/128, stride] for the GEMM.
#include <cuda_fp8.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

constexpr int kMaxEPerLane = 16;  // E <= 512
constexpr int kMaxTopK = 16;

// mode: 0 softmax->topk, 1 sigmoid group-limited, 2 topk->softmax
// One warp routes one token; `row` holds the token's E router logits (global or shared memory).
template <typename T>
__device__ __forceinline__ void route_row(float* __restrict__ out_w, int* __restrict__ out_ids, const T* row,
                                          const float* __restrict__ bias, int64_t t, int lane, int E, int k, int mode,
                                          int renorm, int n_group, int topk_group, float scale) {
  const int per = (E + 31) / 32;
  float score[kMaxEPerLane];  // unbiased weight source
  float sel[kMaxEPerLane];    // selection score
  // expert e lives on lane e % 32, slot e / 32
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < kMaxEPerLane; ++s) {
    int e = s * 32 + lane;
    float v = (s < per && e < E) ? to_f(row[e]) : -INFINITY;
    score[s] = v;
    mx = fmaxf(mx, v);
  }
  if (mode == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxEPerLane; ++s) {
      float p = (score[s] == -INFINITY) ? 0.f : __expf(score[s] - mx);
      sum += p;
      score[s] = p;
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int s = 0; s < kMaxEPerLane; ++s) {
      int e = s * 32 + lane;
      score[s] = (s < per && e < E) ? score[s] / sum : -INFINITY;
      sel[s] = score[s];
    }
  } else if (mode == 1) {
#pragma unroll
    for (int s = 0; s < kMaxEPerLane; ++s) {
      int e = s * 32 + lane;
      bool ok = s < per && e < E;
      float sg = ok ? 1.f / (1.f + __expf(-score[s])) : -INFINITY;
      score[s] = sg;
      sel[s] = ok ? sg + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    if (n_group > 1) {
      // group score = sum of the two best selection scores in the group; keep the best topk_group groups
      const int gsz = E / n_group;
      float gscore_mine = -INFINITY;  // lane g holds the score of group g (n_group <= 32)
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int s = 0; s < kMaxEPerLane; ++s) {
          int e = s * 32 + lane;
          if (s < per && e < E && e / gsz == g) {
            float v = sel[s];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v;
          }
        }
        // merge (b1, b2) pairs across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float o1 = __shfl_xor_sync(0xffffffff, b1, o), o2 = __shfl_xor_sync(0xffffffff, b2, o);
          float n1 = fmaxf(b1, o1);
          float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        float gs = (gsz >= 2) ? b1 + b2 : b1;
        if (lane == g) gscore_mine = gs;
      }
      uint32_t keep = 0;
      for (int r = 0; r < topk_group; ++r) {
        float v = gscore_mine;
        int idx = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float ov = __shfl_xor_sync(0xffffffff, v, o);
          int oi = __shfl_xor_sync(0xffffffff, idx, o);
          if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        keep |= 1u << idx;
        if (lane == idx) gscore_mine = -INFINITY;
      }
#pragma unroll
      for (int s = 0; s < kMaxEPerLane; ++s) {
        int e = s * 32 + lane;
        if (s < per && e < E && !((keep >> (e / gsz)) & 1u)) sel[s] = -INFINITY;
      }
    }
  } else {
#pragma unroll
    for (int s = 0; s < kMaxEPerLane; ++s) sel[s] = score[s];
  }
  // k rounds of warp arg-max over sel
  float wsel[kMaxTopK];
  int isel[kMaxTopK];
  float wsum = 0.f;
  for (int r = 0; r < k; ++r) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    float sc = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxEPerLane; ++s) {
      int e = s * 32 + lane;
      if (s < per && e < E && (sel[s] > v || (sel[s] == v && e < idx))) { v = sel[s]; idx = e; sc = score[s]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffff, v, o);
      int oi = __shfl_xor_sync(0xffffffff, idx, o);
      float os = __shfl_xor_sync(0xffffffff, sc, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; sc = os; }
    }
    wsel[r] = sc;
    isel[r] = idx;
    wsum += sc;
    if (idx != 0x7fffffff && (idx & 31) == lane) sel[idx >> 5] = -INFINITY;
  }
  if (mode == 2) {  // softmax over the selected logits
    float m2 = -INFINITY;
    for (int r = 0; r < k; ++r) m2 = fmaxf(m2, wsel[r]);
    float s2 = 0.f;
    for (int r = 0; r < k; ++r) { wsel[r] = __expf(wsel[r] - m2); s2 += wsel[r]; }
    for (int r = 0; r < k; ++r) wsel[r] /= s2;
  } else if (renorm) {
    float inv = 1.f / (wsum + (mode == 1 ? 1e-20f : 0.f));
    for (int r = 0; r < k; ++r) wsel[r] *= inv;
  }
  if (lane == 0) {
    for (int r = 0; r < k; ++r) {
      out_w[t * k + r] = wsel[r] * (mode == 2 ? 1.f : scale);
      out_ids[t * k + r] = (isel[r] == 0x7fffffff) ? 0 : isel[r];
    }
  }
}


template <typename T>
__global__ void moe_route_kernel(float* __restrict__ out_w, int* __restrict__ out_ids, const T* __restrict__ logits,
                                 const float* __restrict__ bias, int64_t T_, int E, int k, int mode, int renorm,
                                 int n_group, int topk_group, float scale, int64_t stride) {
  griddep_launch();
  griddep_wait();
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  route_row<T>(out_w, out_ids, logits + t * stride, bias, t, threadIdx.x & 31, E, k, mode, renorm, n_group, topk_group,
               scale);
}

// Router GEMM and routing in one launch for decode-sized batches: one CTA per token computes its E logits into
// shared memory (each warp a slice of the experts, 16-byte loads of the router rows), then warp 0 routes the token.
template <typename T>
__global__ void __launch_bounds__(256) router_route_small_kernel(
    float* __restrict__ out_w, int* __restrict__ out_ids, const T* __restrict__ x, int64_t x_stride,
    const T* __restrict__ w, const T* __restrict__ wbias, const float* __restrict__ bias, int E, int K, int k, int mode,
    int renorm, int n_group, int topk_group, float scale) {
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char smem_rr[];
  T* sx = reinterpret_cast<T*>(smem_rr);
  float* slog = reinterpret_cast<float*>(smem_rr + (((size_t)K * sizeof(T) + 15) & ~(size_t)15));
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int i = threadIdx.x * V; i < K; i += blockDim.x * V) st_vec(sx + i, ld_vec(x + (int64_t)t * x_stride + i));
  __syncthreads();
  for (int n = warp; n < E; n += nw) {
    const T* wr = w + (int64_t)n * K;
    float acc = 0.f;
    for (int i = lane * V; i < K; i += 32 * V) {
      Vec16<T> a = ld_vec(wr + i), b = ld_vec(sx + i);
#pragma unroll
      for (int e = 0; e < V; ++e) acc += to_f(a.v[e]) * to_f(b.v[e]);
    }
    acc = warp_sum(acc);
    if (lane == 0) slog[n] = acc + (wbias ? to_f(wbias[n]) : 0.f);
  }
  __syncthreads();
  if (warp == 0) route_row<float>(out_w, out_ids, slog, bias, t, lane, E, k, mode, renorm, n_group, topk_group, scale);
}

// counts[e] += number of pairs routed to local expert e  (counts zeroed by the caller kernel chain)
__global__ void moe_count_kernel(int* __restrict__ counts, const int* __restrict__ ids, const int* __restrict__ emap,
                                 int64_t pairs, int E_local, int E_global) {
  extern __shared__ int sh_cnt[];
  griddep_launch();
  griddep_wait();
  for (int i = threadIdx.x; i < E_local; i += blockDim.x) sh_cnt[i] = 0;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
    int e = ids[i];
    if (e < 0 || e >= E_global) continue;
    if (emap) e = emap[e];
    if (e >= 0 && e < E_local) atomicAdd(&sh_cnt[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E_local; i += blockDim.x)
    if (sh_cnt[i]) atomicAdd(&counts[i], sh_cnt[i]);
}

// lod = exclusive scan of counts; cursor = lod[:-1]; counts re-zeroed for the next call
__global__ void moe_scan_kernel(int* __restrict__ lod, int* __restrict__ cursor, int* __restrict__ counts, int E_local) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x;
  int run = 0;
  for (int e0 = 0; e0 < E_local; e0 += 32) {
    int e = e0 + lane;
    int c = e < E_local ? counts[e] : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffff, inc, o);
      if (lane >= o) inc += v;
    }
    if (e < E_local) { lod[e] = run + inc - c; cursor[e] = run + inc - c; counts[e] = 0; }
    run += __shfl_sync(0xffffffff, inc, 31);
  }
  if (lane == 0) lod[E_local] = run;
}

// One warp per (token, slot) pair: claim a row of the expert's segment and copy the token row there.
template <typename T>
__global__ void moe_scatter_kernel(T* __restrict__ x_sorted, int* __restrict__ pos_of_pair, int* __restrict__ cursor,
                                   const T* __restrict__ x, const int* __restrict__ ids, const int* __restrict__ emap,
                                   int64_t pairs, int k, int H, int E_local, int E_global, int64_t x_stride,
                                   int64_t max_rows) {
  constexpr int V = Vec16<T>::N;
  griddep_launch();
  griddep_wait();
  const int64_t pair = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  int e = ids[pair];
  if (e >= 0 && e < E_global && emap) e = emap[e];
  int pos = -1;
  if (e >= 0 && e < E_local) {
    if (lane == 0) pos = atomicAdd(&cursor[e], 1);
    pos = __shfl_sync(0xffffffff, pos, 0);
    if (pos >= max_rows) pos = -1;
  }
  if (lane == 0) pos_of_pair[pair] = pos;
  if (pos < 0) return;
  const T* src = x + (pair / k) * x_stride;
  T* dst = x_sorted + (int64_t)pos * H;
  for (int i = lane; i < H / V; i += 32) st_vec(dst + i * V, ld_vec(src + i * V));
}

template <typename T>
__global__ void moe_unpermute_kernel(T* __restrict__ out, const T* __restrict__ y_sorted,
                                     const int* __restrict__ pos_of_pair, const float* __restrict__ w, int64_t T_,
                                     int k, int H) {
  constexpr int V = Vec16<T>::N;
  griddep_launch();
  griddep_wait();
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H / V; i += blockDim.x) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      int pos = pos_of_pair[t * k + s];
      if (pos < 0) continue;
      float wt = w[t * k + s];
      Vec16<T> a = ld_vec(y_sorted + (int64_t)pos * H + i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += wt * to_f(a.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = from_f<T>(acc[j]);
    st_vec(out + t * H + i * V, o);
  }
}

// One warp per (row, 128-group): absmax -> scale -> e4m3.  Rows >= *rows_valid_ptr (if given) are skipped.
template <typename T>
__global__ void quant_fp8_group_kernel(uint8_t* __restrict__ q, float* __restrict__ scale_t, const T* __restrict__ x,
                                       int64_t rows, int K, int64_t x_stride, int64_t s_stride, int ue8m0,
                                       const int* __restrict__ rows_valid_ptr) {
  griddep_launch();
  griddep_wait();
  const int groups = K / 128;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * groups) return;
  const int64_t row = w / groups;
  const int g = (int)(w - row * groups);
  if (rows_valid_ptr != nullptr && row >= *rows_valid_ptr) return;
  const int lane = threadIdx.x & 31;
  const T* src = x + row * x_stride + g * 128 + lane * 4;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = to_f(src[j]); amax = fmaxf(amax, fabsf(v[j])); }
  amax = fmaxf(warp_max(amax), 1e-10f);
  float scale = amax / 448.f;
  if (ue8m0) scale = exp2f(ceilf(log2f(scale)));
  const float inv = 1.f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    packed |= (uint32_t)(uint8_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
  reinterpret_cast<uint32_t*>(q + row * (int64_t)K + g * 128)[lane] = packed;
  if (lane == 0) scale_t[(int64_t)g * s_stride + row] = scale;
}


// ---- small batches (decode): permute (+ fp8 quantisation) in ONE launch ----------------------------------------
// With at most kSmallPairs (token, slot) pairs every CTA recomputes the whole schedule in shared memory - expert
// counts, their exclusive scan and, for each pair, its rank among the earlier pairs of the same expert - so that
// positions are deterministic and no global counters or second / third launch are needed.  CTA b then moves the
// pairs b, b + G, ...: a plain row copy, or the 1x128 fp8 quantisation of the row straight into its permuted
// place (scales in the transposed layout the grouped GEMM reads).  Replaces count + scan + scatter (+ quant).
constexpr int kSmallPairs = 1024;

template <typename T, bool kQuant>
__global__ void __launch_bounds__(256) moe_prepare_small_kernel(
    void* __restrict__ x_sorted, float* __restrict__ scale_t, int64_t s_stride, int* __restrict__ pos_of_pair,
    int* __restrict__ lod, const T* __restrict__ x, const int* __restrict__ ids, const int* __restrict__ emap, int pairs,
    int k, int H, int E_local, int E_global, int64_t x_stride) {
  extern __shared__ int sh[];          // [E_local + 1] lod | [pairs] expert of pair | [pairs] position
  int* s_lod = sh;
  int* s_e = sh + E_local + 1;
  int* s_pos = s_e + pairs;
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x;
  for (int i = tid; i <= E_local; i += blockDim.x) s_lod[i] = 0;
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    int e = ids[p];
    if (e >= 0 && e < E_global && emap) e = emap[e];
    if (e < 0 || e >= E_local) e = -1;
    s_e[p] = e;
    if (e >= 0) atomicAdd(&s_lod[e + 1], 1);
  }
  __syncthreads();
  if (tid < 32) {  // inclusive scan of the counts, 32 experts per round
    int run = 0;
    for (int e0 = 0; e0 < E_local; e0 += 32) {
      int e = e0 + tid;
      int c = e < E_local ? s_lod[e + 1] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffff, inc, o);
        if (tid >= o) inc += v;
      }
      if (e < E_local) s_lod[e + 1] = run + inc;
      run += __shfl_sync(0xffffffff, inc, 31);
    }
  }
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int e = s_e[p];
    int pos = -1;
    if (e >= 0) {
      int rank = 0;
      for (int q = 0; q < p; ++q) rank += (s_e[q] == e);
      pos = s_lod[e] + rank;
    }
    s_pos[p] = pos;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int i = tid; i <= E_local; i += blockDim.x) lod[i] = s_lod[i];
    for (int p = tid; p < pairs; p += blockDim.x) pos_of_pair[p] = s_pos[p];
  }
  const int warp = tid >> 5, lane = tid & 31, wpb = blockDim.x >> 5;
  for (int p = blockIdx.x * wpb + warp; p < pairs; p += gridDim.x * wpb) {
    const int pos = s_pos[p];
    if (pos < 0) continue;
    const T* src = x + (int64_t)(p / k) * x_stride;
    if (kQuant) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(x_sorted) + (int64_t)pos * H;
      for (int g = 0; g < H / 128; ++g) {
        float v[4];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[j] = to_f(src[g * 128 + lane * 4 + j]); amax = fmaxf(amax, fabsf(v[j])); }
        amax = fmaxf(warp_max(amax), 1e-10f);
        const float scale = amax / 448.f, inv = 1.f / scale;
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          packed |= (uint32_t)(uint8_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        reinterpret_cast<uint32_t*>(dst + g * 128)[lane] = packed;
        if (lane == 0) scale_t[(int64_t)g * s_stride + pos] = scale;
      }
    } else {
      constexpr int V = Vec16<T>::N;
      T* dst = reinterpret_cast<T*>(x_sorted) + (int64_t)pos * H;
      for (int i = lane; i < H / V; i += 32) st_vec(dst + i * V, ld_vec(src + i * V));
    }
  }
}

// a = act(h[:, :I]) * h[:, I:] quantised to fp8 with 1x128 scales in one pass (rows >= *rows_valid are skipped)
template <typename T>
__global__ void act_mul_quant_fp8_kernel(uint8_t* __restrict__ q, float* __restrict__ scale_t, const T* __restrict__ h,
                                         int64_t rows, int I, int64_t s_stride, int act, const int* __restrict__ rows_valid_ptr) {
  griddep_launch();
  griddep_wait();
  const int groups = I / 128;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * groups) return;
  const int64_t row = w / groups;
  const int g = (int)(w - row * groups);
  if (rows_valid_ptr != nullptr && row >= *rows_valid_ptr) return;
  const int lane = threadIdx.x & 31;
  const T* gp = h + row * 2 * (int64_t)I + g * 128 + lane * 4;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float gf = to_f(gp[j]), uf = to_f(gp[I + j]);
    float a;
    if (act == 0) a = gf / (1.f + __expf(-gf));
    else { float t = 0.7978845608f * (gf + 0.044715f * gf * gf * gf); a = 0.5f * gf * (1.f + tanhf(t)); }
    // round through T exactly like the two-kernel path (activation kernel output, then quantiser input)
    v[j] = to_f(from_f<T>(a * uf));
    amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = fmaxf(warp_max(amax), 1e-10f);
  const float scale = amax / 448.f, inv = 1.f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    packed |= (uint32_t)(uint8_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
  reinterpret_cast<uint32_t*>(q + row * (int64_t)I + g * 128)[lane] = packed;
  if (lane == 0) scale_t[(int64_t)g * s_stride + row] = scale;
}


// ---- router GEMM for decode-sized batches -------------------------------------------------------------------
// logits[t, n] = x[t] . w[n] (+ bias[n]) in fp32 for a handful of tokens and at most a few hundred experts: far too
// small for the tensor-core GEMM, whose fixed cost (TMEM, barriers, pipeline fill, split-K fix-up) is ~10 us.
// One CTA per (token, 32 experts): the activation row sits in shared memory, each warp produces 4 logits with
// 16-byte loads of the weight rows.  (GateLinear's small-batch tier, ops/fused_moe/router/gate_linear.py:37-116.)
template <typename T>
__global__ void __launch_bounds__(256) router_gemm_small_kernel(float* __restrict__ out, const T* __restrict__ x,
                                                                int64_t x_stride, const T* __restrict__ w,
                                                                const T* __restrict__ bias, int N, int K) {
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char smem_router[];
  T* sx = reinterpret_cast<T*>(smem_router);
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, n0 = blockIdx.y * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x * V; i < K; i += blockDim.x * V) st_vec(sx + i, ld_vec(x + (int64_t)t * x_stride + i));
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + warp * 4 + j;
    if (n >= N) break;
    const T* wr = w + (int64_t)n * K;
    float acc = 0.f;
    for (int i = lane * V; i < K; i += 32 * V) {
      Vec16<T> a = ld_vec(wr + i), b = ld_vec(sx + i);
#pragma unroll
      for (int e = 0; e < V; ++e) acc += to_f(a.v[e]) * to_f(b.v[e]);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(int64_t)t * N + n] = acc + (bias ? to_f(bias[n]) : 0.f);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route(float* out_w, int* out_ids, const void* logits, const float* bias, int64_t T_, int E,
                              int k, int mode, int renorm, int n_group, int topk_group, float scale, int64_t stride,
                              int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  if (E > 32 * kMaxEPerLane || k > kMaxTopK || n_group > 32 || (n_group > 1 && E % n_group)) return 2;
  const int wpb = 4;
  B200_DISPATCH_DTYPE(dtype, {
    launch_pdl(moe_route_kernel<T>, dim3((T_ + wpb - 1) / wpb), dim3(wpb * 32), 0, st, out_w, out_ids,
               (const T*)logits, bias, T_, E, k, mode, renorm, n_group, topk_group, scale, stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_moe_permute(void* x_sorted, int* pos_of_pair, int* lod, int* counts, int* cursor, const void* x,
                                const int* ids, const int* emap, int64_t T_, int k, int H, int E_local, int E_global,
                                int64_t x_stride, int64_t max_rows, int dtype, cudaStream_t st) {
  const int64_t pairs = T_ * k;
  int blocks = (int)((pairs + 255) / 256);
  if (blocks > 256) blocks = 256;
  if (blocks < 1) blocks = 1;
  launch_pdl(moe_count_kernel, dim3(blocks), dim3(256), (size_t)E_local * sizeof(int), st, counts, ids, emap, pairs,
             E_local, E_global);
  launch_pdl(moe_scan_kernel, dim3(1), dim3(32), 0, st, lod, cursor, counts, E_local);
  if (pairs > 0) {
    B200_DISPATCH_DTYPE(dtype, {
      if (H % Vec16<T>::N) return 2;
      launch_pdl(moe_scatter_kernel<T>, dim3((pairs + 7) / 8), dim3(256), 0, st, (T*)x_sorted, pos_of_pair, cursor,
                 (const T*)x, ids, emap, pairs, k, H, E_local, E_global, x_stride, max_rows);
    });
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_moe_unpermute(void* out, const void* y_sorted, const int* pos_of_pair, const float* w, int64_t T_,
                                  int k, int H, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    if (H % Vec16<T>::N) return 2;
    launch_pdl(moe_unpermute_kernel<T>, dim3(T_), dim3(256), 0, st, (T*)out, (const T*)y_sorted, pos_of_pair, w, T_,
               k, H);
  });
  return (int)cudaGetLastError();
}

// Per-token int8 quantisation of activations (compressed-tensors W8A8; reference: quantization/kernels/
// scale_mm.py:43-90).  Dynamic: scale[t] = max|x[t]| / 127; static: the given per-tensor scale.  One warp per row.
template <typename T>
__global__ void quant_int8_token_kernel(int8_t* __restrict__ q, float* __restrict__ scale, const T* __restrict__ x,
                                        const float* __restrict__ static_scale, int64_t rows, int K, int64_t x_stride) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* src = x + row * x_stride;
  float s;
  if (static_scale != nullptr) {
    s = static_scale[0];
  } else {
    float amax = 0.f;
    for (int i = lane; i < K; i += 32) amax = fmaxf(amax, fabsf(to_f(src[i])));
    s = fmaxf(warp_max(amax), 1e-8f) / 127.f;
  }
  if (lane == 0) scale[row] = s;
  for (int i = lane; i < K; i += 32) {
    const float v = rintf(to_f(src[i]) / s);
    q[row * K + i] = (int8_t)fminf(fmaxf(v, -128.f), 127.f);
  }
}

extern "C" int b200_quant_int8_token(void* q, float* scale, const void* x, const float* static_scale, int64_t rows,
                                     int K, int64_t x_stride, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    quant_int8_token_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>((int8_t*)q, scale, (const T*)x, static_scale,
                                                                         rows, K, x_stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_quant_fp8_group(void* q, float* scale_t, const void* x, int64_t rows, int K, int64_t x_stride,
                                    int64_t s_stride, int ue8m0, const int* rows_valid_ptr, int dtype,
                                    cudaStream_t st) {
  if (rows == 0) return 0;
  if (K % 128) return 2;
  const int64_t warps = rows * (K / 128);
  B200_DISPATCH_DTYPE(dtype, {
    launch_pdl(quant_fp8_group_kernel<T>, dim3((warps + 7) / 8), dim3(256), 0, st, (uint8_t*)q, scale_t, (const T*)x,
               rows, K, x_stride, s_stride, ue8m0, rows_valid_ptr);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_moe_small_pairs() { return kSmallPairs; }

extern "C" int b200_moe_prepare_small(void* x_sorted, float* scale_t, int64_t s_stride, int* pos_of_pair, int* lod,
                                      const void* x, const int* ids, const int* emap, int64_t T_, int k, int H, int E_local,
                                      int E_global, int64_t x_stride, int quant, int dtype, cudaStream_t st) {
  const int pairs = (int)(T_ * k);
  if (pairs > kSmallPairs || pairs < 1 || (quant && H % 128)) return 2;
  const size_t smem = (size_t)(E_local + 1 + 2 * pairs) * sizeof(int);
  int grid = (pairs + 7) / 8;
  if (grid > 64) grid = 64;
  B200_DISPATCH_DTYPE(dtype, {
    if (H % Vec16<T>::N) return 2;
    if (quant)
      launch_pdl(moe_prepare_small_kernel<T, true>, dim3(grid), dim3(256), smem, st, x_sorted, scale_t, s_stride, pos_of_pair,
                 lod, (const T*)x, ids, emap, pairs, k, H, E_local, E_global, x_stride);
    else
      launch_pdl(moe_prepare_small_kernel<T, false>, dim3(grid), dim3(256), smem, st, x_sorted, scale_t, s_stride,
                 pos_of_pair, lod, (const T*)x, ids, emap, pairs, k, H, E_local, E_global, x_stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_act_mul_quant_fp8(void* q, float* scale_t, const void* h, int64_t rows, int I, int64_t s_stride, int act,
                                      const int* rows_valid_ptr, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (I % 128 || act > 1) return 2;
  const int64_t warps = rows * (I / 128);
  B200_DISPATCH_DTYPE(dtype, {
    launch_pdl(act_mul_quant_fp8_kernel<T>, dim3((warps + 7) / 8), dim3(256), 0, st, (uint8_t*)q, scale_t, (const T*)h, rows,
               I, s_stride, act, rows_valid_ptr);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_router_gemm_small(float* out, const void* x, int64_t x_stride, const void* w, const void* bias,
                                      int64_t T_, int N, int K, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  int esz = dtype == 0 ? 4 : 2;
  if (K % (16 / esz) || (x_stride * esz) % 16 || (size_t)K * esz > 96 * 1024) return 2;
  B200_DISPATCH_DTYPE(dtype, {
    if ((size_t)K * esz > 48 * 1024) ensure_dynamic_smem((const void*)router_gemm_small_kernel<T>, 96 * 1024);
    launch_pdl(router_gemm_small_kernel<T>, dim3((unsigned)T_, (N + 31) / 32), dim3(256), (size_t)K * esz, st, out,
               (const T*)x, x_stride, (const T*)w, (const T*)bias, N, K);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_router_route_small(float* out_w, int* out_ids, const void* x, int64_t x_stride, const void* w,
                                       const void* wbias, const float* bias, int64_t T_, int E, int K, int k, int mode,
                                       int renorm, int n_group, int topk_group, float scale, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  if (E > 32 * kMaxEPerLane || k > kMaxTopK || n_group > 32 || (n_group > 1 && E % n_group)) return 2;
  const int esz = dtype == 0 ? 4 : 2;
  if (K % (16 / esz) || (x_stride * esz) % 16) return 2;
  const size_t smem = (((size_t)K * esz + 15) & ~(size_t)15) + (size_t)E * 4;
  if (smem > 96 * 1024) return 2;
  B200_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024) ensure_dynamic_smem((const void*)router_route_small_kernel<T>, 96 * 1024);
    launch_pdl(router_route_small_kernel<T>, dim3((unsigned)T_), dim3(256), smem, st, out_w, out_ids, (const T*)x,
               x_stride, (const T*)w, (const T*)wbias, bias, E, K, k, mode, renorm, n_group, topk_group, scale);
  });
  return (int)cudaGetLastError();
}
