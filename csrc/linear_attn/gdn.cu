// Gated DeltaNet (Qwen3-Next linear-attention layers) device ops: varlen causal conv1d with a state
// cache, single-token conv update, gating, and the gated delta rule as a sequential scan that keeps the
// [Dv, Dk] state of one head in registers.
//
// Reference entry points: kunlun_ops.causal_conv1d_fn / causal_conv1d_update
// (vllm_kunlun/ops/mamba/causal_conv1d.py:15-74,118-225), fused_gdn_gating (models/qwen3_next.py:262-781),
// fused_recurrent_gated_delta_rule (ops/fla/fused_recurrent.py:52-155) and the chunked form
// (ops/fla/chunk.py:23-140), which is numerically the same recurrence.
#include "../api.h"
#include "../common/utils.cuh"

namespace b200 {
namespace {

constexpr int kMaxW = 8;

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

__device__ __forceinline__ int find_seq(const int* __restrict__ cu, int R, int t) {
  int lo = 0, hi = R;  // largest r with cu[r] <= t
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// y[t, c] = act(bias[c] + sum_j w[c, j] * in[t - (W-1) + j, c]); positions before the sequence start read
// the cached state (rows W-1+p.. of the previous inputs) or zero.
// One thread = one 16-byte channel vector x kConvTok consecutive tokens, with a sliding window of the last W-1
// input rows in registers, so every input row is loaded once per thread.
constexpr int kConvTok = 8;

template <typename T, int W>
__global__ void __launch_bounds__(128) conv1d_fwd_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x,
                                                         int64_t x_stride, const T* __restrict__ w, const T* __restrict__ bias,
                                                         const int* __restrict__ cu, int R, const T* __restrict__ states,
                                                         const int* __restrict__ slots, const uint8_t* __restrict__ has_init,
                                                         int C, int act, int64_t Ttot) {
  constexpr int V = Vec16<T>::N;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  const int64_t t0 = (int64_t)blockIdx.y * kConvTok;
  if (c0 >= C || t0 >= Ttot) return;
  float wv[W][V], bv[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    bv[e] = bias ? to_f(bias[c0 + e]) : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) wv[j][e] = to_f(w[(int64_t)(c0 + e) * W + j]);
  }
  float win[W][V];  // win[j] = input row at (current token) - (W-1) + j
  int r = find_seq(cu, R, (int)t0);
  int seq_start = cu[r], seq_end = cu[r + 1];
  auto load_hist = [&](int64_t t) {  // fill win[0 .. W-2] with the W-1 rows in front of token t
    const int p = (int)t - seq_start;
    const int slot = slots[r];
    const bool init = has_init[r] != 0 && slot >= 0;
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      const int q = p - (W - 1) + j;
      if (q >= 0) {
        Vec16<T> v = ld_vec(x + (t - (W - 1) + j) * x_stride + c0);
#pragma unroll
        for (int e = 0; e < V; ++e) win[j][e] = to_f(v.v[e]);
      } else if (init) {
        Vec16<T> v = ld_vec(states + ((int64_t)slot * (W - 1) + (W - 1 + q)) * C + c0);
#pragma unroll
        for (int e = 0; e < V; ++e) win[j][e] = to_f(v.v[e]);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) win[j][e] = 0.f;
      }
    }
  };
  load_hist(t0);
  for (int i = 0; i < kConvTok; ++i) {
    const int64_t t = t0 + i;
    if (t >= Ttot) break;
    if (t >= seq_end) {  // crossed into the next (non-empty) sequence: its history comes from its own state
      while (t >= seq_end) { ++r; seq_start = cu[r]; seq_end = cu[r + 1]; }
      load_hist(t);
    }
    Vec16<T> cur = ld_vec(x + t * x_stride + c0);
    Vec16<T> o;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      win[W - 1][e] = to_f(cur.v[e]);
      float acc = bv[e];
#pragma unroll
      for (int j = 0; j < W; ++j) acc += wv[j][e] * win[j][e];
      o.v[e] = from_f<T>(act ? silu(acc) : acc);
    }
    st_vec(out + t * out_stride + c0, o);
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
#pragma unroll
      for (int e = 0; e < V; ++e) win[j][e] = win[j + 1][e];
    }
  }
}

// states[slot] <- last W-1 rows of (old state ++ x[seq]); one thread owns a channel column.
template <typename T>
__global__ void conv1d_state_kernel(T* __restrict__ states, const T* __restrict__ x, int64_t x_stride,
                                    const int* __restrict__ cu, const int* __restrict__ slots,
                                    const uint8_t* __restrict__ has_init, int C, int W) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= C) return;
  const int s = cu[r], L = cu[r + 1] - s, slot = slots[r];
  if (L == 0 || slot < 0) return;
  const bool init = has_init[r] != 0;
  float keep[kMaxW];
  for (int j = 0; j < W - 1; ++j) {
    const int q = L - (W - 1) + j;
    if (q >= 0) keep[j] = to_f(x[(int64_t)(s + q) * x_stride + c]);
    else keep[j] = init ? to_f(states[((int64_t)slot * (W - 1) + (W - 1 + q)) * C + c]) : 0.f;
  }
  for (int j = 0; j < W - 1; ++j) states[((int64_t)slot * (W - 1) + j) * C + c] = from_f<T>(keep[j]);
}

template <typename T>
__global__ void conv1d_update_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x, int64_t x_stride,
                                     T* __restrict__ states, const T* __restrict__ w, const T* __restrict__ bias,
                                     const int* __restrict__ slots, int C, int W, int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int slot = slots[b];
  if (slot < 0) { out[(int64_t)b * out_stride + c] = from_f<T>(0.f); return; }
  T* st = states + (int64_t)slot * (W - 1) * C + c;
  float acc = bias ? to_f(bias[c]) : 0.f;
  float cur = to_f(x[(int64_t)b * x_stride + c]);
  for (int j = 0; j < W - 1; ++j) {
    float v = to_f(st[(int64_t)j * C]);
    acc += to_f(w[(int64_t)c * W + j]) * v;
    if (j > 0) st[(int64_t)(j - 1) * C] = from_f<T>(v);
  }
  acc += to_f(w[(int64_t)c * W + W - 1]) * cur;
  st[(int64_t)(W - 2) * C] = from_f<T>(cur);
  out[(int64_t)b * out_stride + c] = from_f<T>(act ? silu(acc) : acc);
}

// g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b)
template <typename T>
__global__ void gdn_gating_kernel(float* __restrict__ g, float* __restrict__ beta, const T* __restrict__ a, int64_t a_stride,
                                  const T* __restrict__ b, int64_t b_stride, const float* __restrict__ A_log,
                                  const float* __restrict__ dt_bias, int H, int64_t T_) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= T_ * H) return;
  int64_t t = i / H;
  int h = (int)(i % H);
  float xa = to_f(a[t * a_stride + h]) + dt_bias[h];
  float sp = xa > 20.f ? xa : log1pf(__expf(xa));
  g[i] = -__expf(A_log[h]) * sp;
  beta[i] = 1.f / (1.f + __expf(-to_f(b[t * b_stride + h])));
}

// Sequential gated delta rule.  Block = 128 threads = 32 state rows (of Dv) x 4 quarters of Dk; grid
// (Dv/32, Hv, sequences).  Per token: S *= exp(g); pred = S k; S += beta (v - pred) k^T; o = S q.
// Tokens are staged through shared memory in chunks of kGdnChunk: while the block works through one chunk
// (no block-wide barrier inside: a row's four quarter-threads are adjacent lanes), every thread already holds its
// share of the next chunk's q / k / v / g / beta in registers, so global-memory latency never sits on the
// recurrence and the block synchronises twice per chunk instead of once per token.
constexpr int kGdnChunk = 16;

template <typename T, int DK>
__global__ void __launch_bounds__(128) gdn_recurrent_kernel(
    T* __restrict__ out, int64_t o_stride, const T* __restrict__ q, const T* __restrict__ k, int64_t qk_stride,
    const T* __restrict__ v, int64_t v_stride, const float* __restrict__ g, const float* __restrict__ beta,
    float* __restrict__ states /*[slots, Hv, Dv, DK]*/, const int* __restrict__ cu, const int* __restrict__ slots,
    const uint8_t* __restrict__ has_init, int Hk, int Hv, int Dv, float scale, int l2norm) {
  static_assert(DK % 16 == 0 && DK <= 128, "DK");
  constexpr int QW = DK / 4;                      // state columns per thread
  constexpr int CH = kGdnChunk;
  constexpr int QK_PER = CH * DK / 128;           // q (and k) elements of a chunk per thread
  constexpr int V_PER = CH * 32 / 128;            // v elements of a chunk per thread
  __shared__ __align__(16) float sk[CH][DK];
  __shared__ __align__(16) float sq[CH][DK];
  __shared__ float sv[CH][32];
  __shared__ float sg[CH], sb[CH], srk[CH], srq[CH];
  const int tid = threadIdx.x, rl = tid >> 2, qd = tid & 3, warp = tid >> 5, lane = tid & 31;
  const int hv = blockIdx.y, r = blockIdx.z, hk = hv / (Hv / Hk);
  const int row0 = blockIdx.x * 32, row = row0 + rl;
  const int s = cu[r], L = cu[r + 1] - s, slot = slots[r];
  if (L == 0 || slot < 0) return;
  // Column ownership is interleaved in 16-byte pieces: registers S[4i .. 4i+3] of quarter qd hold columns
  // 16 i + 4 qd .. + 3, so that the four quarter-lanes of a row read four consecutive float4 of the shared k / q row
  // (distinct banks) instead of four addresses 128 bytes apart (one bank, a 4-way conflict on every load).
  float* sp = states + (((int64_t)slot * Hv + hv) * Dv + row) * DK + qd * 4;
  float S[QW];
  if (has_init[r]) {
#pragma unroll
    for (int j = 0; j < QW; j += 4) *reinterpret_cast<float4*>(&S[j]) = *reinterpret_cast<const float4*>(sp + j * 4);
  } else {
#pragma unroll
    for (int j = 0; j < QW; ++j) S[j] = 0.f;
  }
  // register staging of one chunk: element e of the flattened [CH, DK] (resp. [CH, 32]) tile, e = i * 128 + tid
  float rk_[QK_PER], rq_[QK_PER], rv_[V_PER], rg = 0.f, rb = 0.f;
  auto fetch = [&](int c0) {
#pragma unroll
    for (int i = 0; i < QK_PER; ++i) {
      const int e = i * 128 + tid, t = e / DK, d = e % DK;
      const bool ok = c0 + t < L;
      const int64_t tok = s + c0 + t;
      rk_[i] = ok ? to_f(k[tok * qk_stride + hk * DK + d]) : 0.f;
      rq_[i] = ok ? to_f(q[tok * qk_stride + hk * DK + d]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < V_PER; ++i) {
      const int e = i * 128 + tid, t = e / 32, d = e % 32;
      rv_[i] = (c0 + t < L) ? to_f(v[(int64_t)(s + c0 + t) * v_stride + hv * Dv + row0 + d]) : 0.f;
    }
    if (tid < CH && c0 + tid < L) {
      rg = g[(int64_t)(s + c0 + tid) * Hv + hv];
      rb = beta[(int64_t)(s + c0 + tid) * Hv + hv];
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < L; c0 += CH) {
    __syncthreads();  // the previous chunk has been consumed
#pragma unroll
    for (int i = 0; i < QK_PER; ++i) {
      const int e = i * 128 + tid;
      sk[e / DK][e % DK] = rk_[i];
      sq[e / DK][e % DK] = rq_[i];
    }
#pragma unroll
    for (int i = 0; i < V_PER; ++i) {
      const int e = i * 128 + tid;
      sv[e / 32][e % 32] = rv_[i];
    }
    if (tid < CH) { sg[tid] = __expf(rg); sb[tid] = rb; }
    __syncthreads();
    // squared norms: warp w handles tokens w, w + 4, ...
    for (int t = warp; t < CH; t += 4) {
      float k2 = 0.f, q2 = 0.f;
      for (int d = lane; d < DK; d += 32) { k2 += sk[t][d] * sk[t][d]; q2 += sq[t][d] * sq[t][d]; }
      k2 = warp_sum(k2);
      q2 = warp_sum(q2);
      if (lane == 0) {
        srk[t] = l2norm ? rsqrtf(k2 + 1e-6f) : 1.f;
        srq[t] = l2norm ? scale * rsqrtf(q2 + 1e-6f) : scale;
      }
    }
    if (c0 + CH < L) fetch(c0 + CH);  // next chunk's global loads fly while this one is processed
    __syncthreads();
    const int n = min(CH, L - c0);
    for (int t = 0; t < n; ++t) {
      const float gt = sg[t], bt = sb[t], vt = sv[t][rl], rk = srk[t], rq = srq[t];
      const float* kk = &sk[t][qd * 4];
      const float* qq = &sq[t][qd * 4];
      float pred = 0.f, pred2 = 0.f;
#pragma unroll
      for (int j = 0; j < QW; j += 4) {
        float4 k4 = *reinterpret_cast<const float4*>(kk + j * 4);
        S[j] *= gt; S[j + 1] *= gt; S[j + 2] *= gt; S[j + 3] *= gt;
        pred += S[j] * k4.x + S[j + 1] * k4.y;
        pred2 += S[j + 2] * k4.z + S[j + 3] * k4.w;
      }
      pred += pred2;
      pred += __shfl_xor_sync(0xffffffff, pred, 1);
      pred += __shfl_xor_sync(0xffffffff, pred, 2);
      const float delta = (vt - pred * rk) * bt * rk;
      float o = 0.f, o2 = 0.f;
#pragma unroll
      for (int j = 0; j < QW; j += 4) {
        float4 k4 = *reinterpret_cast<const float4*>(kk + j * 4);
        float4 q4 = *reinterpret_cast<const float4*>(qq + j * 4);
        S[j] += delta * k4.x; S[j + 1] += delta * k4.y; S[j + 2] += delta * k4.z; S[j + 3] += delta * k4.w;
        o += S[j] * q4.x + S[j + 1] * q4.y;
        o2 += S[j + 2] * q4.z + S[j + 3] * q4.w;
      }
      o += o2;
      o += __shfl_xor_sync(0xffffffff, o, 1);
      o += __shfl_xor_sync(0xffffffff, o, 2);
      if (qd == 0) out[(int64_t)(s + c0 + t) * o_stride + hv * Dv + row] = from_f<T>(o * rq);
    }
  }
#pragma unroll
  for (int j = 0; j < QW; j += 4) *reinterpret_cast<float4*>(sp + j * 4) = *reinterpret_cast<const float4*>(&S[j]);
}

// MTP input glue: out[t] = [rmsnorm(embed[t]) * (pos != 0), rmsnorm(hidden[t])]  (deepseek_mtp.py:79-87)
template <typename T>
__global__ void mtp_concat_norm_kernel(T* __restrict__ out, const T* __restrict__ embed, const T* __restrict__ hidden,
                                       const T* __restrict__ we, const T* __restrict__ wh, const int64_t* __restrict__ pos,
                                       int H, float eps) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const bool zero = pos && pos[t] == 0;
  float se = 0.f, sh = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float e = zero ? 0.f : to_f(embed[t * H + i]), h = to_f(hidden[t * H + i]);
    se += e * e;
    sh += h * h;
  }
  se = block_sum(se, red);
  sh = block_sum(sh, red);
  const float re = rsqrtf(se / H + eps), rh = rsqrtf(sh / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float e = zero ? 0.f : to_f(embed[t * H + i]), h = to_f(hidden[t * H + i]);
    out[t * 2 * H + i] = from_f<T>(e * re * to_f(we[i]));
    out[t * 2 * H + H + i] = from_f<T>(h * rh * to_f(wh[i]));
  }
}

// out[t, i] = o[t, i] * sigmoid(gate[t, i]) with a strided gate (column slice of a fused projection)
template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ out, const T* __restrict__ o, const T* __restrict__ gate,
                                        int64_t gate_stride, int D, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t t = i / D;
  int c = (int)(i % D);
  float gv = to_f(gate[t * gate_stride + c]);
  out[i] = from_f<T>(to_f(o[i]) / (1.f + __expf(-gv)));
}

}  // namespace
}  // namespace b200

namespace b200 {
namespace {
template <typename T>
int launch_conv_fwd(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* w, const void* bias,
                    const int* cu, int R, void* states, const int* slots, const uint8_t* has_init, int C, int W, int act,
                    int64_t T_, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (C % V != 0 || (x_stride % V) != 0 || (out_stride % V) != 0) return 3;
  dim3 g1((C / V + 127) / 128, (unsigned)((T_ + kConvTok - 1) / kConvTok)), g2((C + 255) / 256, R);
#define B200_CONV_W(WW)                                                                                                   \
  conv1d_fwd_kernel<T, WW><<<g1, 128, 0, st>>>((T*)out, out_stride, (const T*)x, x_stride, (const T*)w, (const T*)bias, cu, \
                                               R, (const T*)states, slots, has_init, C, act, T_)
  switch (W) {
    case 2: B200_CONV_W(2); break;
    case 3: B200_CONV_W(3); break;
    case 4: B200_CONV_W(4); break;
    case 5: B200_CONV_W(5); break;
    case 6: B200_CONV_W(6); break;
    case 7: B200_CONV_W(7); break;
    default: B200_CONV_W(8); break;
  }
#undef B200_CONV_W
  conv1d_state_kernel<T><<<g2, 256, 0, st>>>((T*)states, (const T*)x, x_stride, cu, slots, has_init, C, W);
  return cudaGetLastError() != cudaSuccess;
}
}  // namespace
}  // namespace b200

extern "C" int b200_causal_conv1d_fwd(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* w,
                                      const void* bias, const int* cu, int R, void* states, const int* slots,
                                      const uint8_t* has_init, int C, int W, int act, int64_t T_, int dtype, cudaStream_t st) {
  if (W > b200::kMaxW || W < 2) return 3;
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, return (b200::launch_conv_fwd<T>(out, out_stride, x, x_stride, w, bias, cu, R, states, slots,
                                                              has_init, C, W, act, T_, st)));
  return 1;
}

extern "C" int b200_causal_conv1d_update(void* out, int64_t out_stride, const void* x, int64_t x_stride, void* states,
                                         const void* w, const void* bias, const int* slots, int64_t B, int C, int W, int act,
                                         int dtype, cudaStream_t st) {
  if (W > b200::kMaxW || W < 2) return 3;
  if (B == 0) return 0;
  dim3 g((C + 255) / 256, (unsigned)B);
  B200_DISPATCH_DTYPE(dtype, (b200::conv1d_update_kernel<T><<<g, 256, 0, st>>>((T*)out, out_stride, (const T*)x, x_stride,
                                                                              (T*)states, (const T*)w, (const T*)bias, slots,
                                                                              C, W, act)));
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_gdn_gating(float* g, float* beta, const void* a, int64_t a_stride, const void* b, int64_t b_stride,
                               const float* A_log, const float* dt_bias, int H, int64_t T_, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  unsigned blocks = (unsigned)((T_ * H + 255) / 256);
  B200_DISPATCH_DTYPE(dtype, (b200::gdn_gating_kernel<T><<<blocks, 256, 0, st>>>(g, beta, (const T*)a, a_stride, (const T*)b,
                                                                                 b_stride, A_log, dt_bias, H, T_)));
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_gdn_recurrent(void* out, int64_t o_stride, const void* q, const void* k, int64_t qk_stride, const void* v,
                                  int64_t v_stride, const float* g, const float* beta, float* states, const int* cu,
                                  const int* slots, const uint8_t* has_init, int R, int Hk, int Hv, int Dk, int Dv, float scale,
                                  int l2norm, int dtype, cudaStream_t st) {
  if (R == 0) return 0;
  if (Dv % 32 != 0 || Hv % Hk != 0) return 3;
  dim3 grid(Dv / 32, Hv, R);
#define B200_GDN_LAUNCH(DK)                                                                                          \
  B200_DISPATCH_DTYPE(dtype, (b200::gdn_recurrent_kernel<T, DK><<<grid, 128, 0, st>>>(                                  \
                                 (T*)out, o_stride, (const T*)q, (const T*)k, qk_stride, (const T*)v, v_stride, g, beta, \
                                 states, cu, slots, has_init, Hk, Hv, Dv, scale, l2norm)))
  if (Dk == 128) { B200_GDN_LAUNCH(128); }
  else if (Dk == 64) { B200_GDN_LAUNCH(64); }
  else if (Dk == 32) { B200_GDN_LAUNCH(32); }
  else if (Dk == 16) { B200_GDN_LAUNCH(16); }
  else return 3;
#undef B200_GDN_LAUNCH
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_mtp_concat_norm(void* out, const void* embed, const void* hidden, const void* we, const void* wh,
                                    const int64_t* pos, int64_t T_, int H, float eps, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, (b200::mtp_concat_norm_kernel<T><<<(unsigned)T_, 512, 0, st>>>(
                                 (T*)out, (const T*)embed, (const T*)hidden, (const T*)we, (const T*)wh, pos, H, eps)));
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_sigmoid_gate_mul(void* out, const void* o, const void* gate, int64_t gate_stride, int D, int64_t T_,
                                     int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  int64_t n = T_ * D;
  B200_DISPATCH_DTYPE(dtype, (b200::sigmoid_gate_mul_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
                                 (T*)out, (const T*)o, (const T*)gate, gate_stride, D, n)));
  return cudaGetLastError() != cudaSuccess;
}
