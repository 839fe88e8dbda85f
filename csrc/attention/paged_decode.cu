// Paged GQA decode attention (q_len * group <= 16 packed rows per KV head), split-KV.
//
// One CTA = kWarps warps serves one (request, kv head, kv split).  Each warp streams its own
// 16-key tiles (tile i of the split goes to warp i % kWarps) through a private multi-stage
// cp.async ring and keeps a private online-softmax state, so no block-wide barrier sits inside the
// KV loop: warps drift apart and hide each other's memory latency.  A 16-key tile never straddles
// a cache block (block_size is a multiple of 16), so one block-table lookup serves the tile.
// The per-warp states are merged through shared memory at the end; split partials go to the
// fp32 workspace consumed by merge_splits_kernel.
#include "../api.h"
#include "../common/launch.cuh"
#include <stdlib.h>

#include "attn_common.cuh"

namespace b200 {

constexpr int kDecTile = 16;

// Arrival counters of the split CTAs of one (request, kv head, row tile); zero between launches (the merging CTA
// resets its counter).  One launch at a time per device uses them: concurrent decode-attention launches on
// different streams must not share a device.
constexpr int kMaxTickets = 1 << 18;
static __device__ int g_decode_tickets[kMaxTickets];

template <typename T, int D, int kWarps, int kStages>
__global__ void __launch_bounds__(kWarps * 32) paged_decode_kernel(AttnParams p) {
  constexpr int CH = D / 8;   // 16-byte chunks per row
  constexpr int DT = D / 8;   // O n-tiles
  constexpr int KS = D / 16;  // k-steps of QK^T
  constexpr int kTileElems = kDecTile * D;
  using MT = MmaTraits<T>;
  extern __shared__ __align__(16) uint8_t smem_dec[];
  T* sQ = reinterpret_cast<T*>(smem_dec);  // [16][D]
  T* sKV = sQ + 16 * D;                    // [kWarps][kStages][2][16][D]

  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = p.Hq / p.Hkv;
  const int kvh = blockIdx.y;
  const int req = blockIdx.z / p.num_splits;
  const int split = blockIdx.z % p.num_splits;
  const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
  const int seq_len = p.seq_lens[req];
  const int rows_total = q_len * g;
  const int row0 = blockIdx.x * 16;
  if (row0 >= rows_total || q_len <= 0) return;
  const int ctx = seq_len - q_len;
  const int tok_lo = row0 / g;
  const int tok_hi = min(q_len - 1, (row0 + 15) / g);
  const int kv_end = min(seq_len, ctx + tok_hi + 1);
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, ctx + tok_lo - p.window + 1) / kDecTile * kDecTile;
  const int n_tiles_all = (kv_end - kv_begin + kDecTile - 1) / kDecTile;
  const int tiles_per_split = (n_tiles_all + p.num_splits - 1) / p.num_splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(n_tiles_all, tile_lo + tiles_per_split);
  // tiles of this warp: tile_lo + warp, + kWarps, ...
  const int my_tiles = (tile_hi - tile_lo - warp + kWarps - 1) / kWarps;  // may be <= 0

  const T* q_base = reinterpret_cast<const T*>(p.q);
  const T* kv_base = reinterpret_cast<const T*>(p.kv_cache);
  const int* bt = p.block_tables + (int64_t)req * p.max_blocks;
  const int64_t v_off = (int64_t)p.Hkv * p.block_size * D;

  // ---- Q tile (shared by all warps)
  for (int c = tid; c < 16 * CH; c += kWarps * 32) {
    int r = c / CH, ch = c % CH;
    int prow = row0 + r;
    bool valid = prow < rows_total;
    int tok = valid ? prow / g : 0, hh = valid ? prow % g : 0;
    const T* src = q_base + ((int64_t)(qs + tok) * p.Hq + kvh * g + hh) * D + ch * 8;
    cp_async16(sQ + swz<D>(r, ch), src, valid);
  }
  cp_async_commit();

  T* my_kv = sKV + (size_t)warp * kStages * 2 * kTileElems;
  auto load_tile = [&](int i, int stage) {
    const int base = kv_begin + (tile_lo + warp + i * kWarps) * kDecTile;  // multiple of 16
    const int bi = base / p.block_size;
    int64_t blk = (bi < p.max_blocks) ? bt[bi] : -1;
    const bool blk_ok = blk >= 0 && blk < p.num_blocks;
    if (!blk_ok) blk = 0;
    const int off0 = base % p.block_size;
    const T* srcK0 = kv_base + (((blk * 2) * p.Hkv + kvh) * p.block_size + off0) * (int64_t)D;
    T* dK = my_kv + stage * 2 * kTileElems;
    T* dV = dK + kTileElems;
#pragma unroll
    for (int c = lane; c < kDecTile * CH; c += 32) {
      int r = c / CH, ch = c % CH;
      bool valid = blk_ok && (base + r < kv_end);
      const T* s = srcK0 + (valid ? r * D + ch * 8 : 0);
      cp_async16(dK + swz<D>(r, ch), s, valid);
      cp_async16(dV + swz<D>(r, ch), s + v_off, valid);
    }
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < my_tiles) load_tile(s, s);
    cp_async_commit();
  }

  // Q fragments live in registers for the whole KV loop.
  cp_async_wait<kStages - 1>();
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    int r = (lane & 7) + ((lane >> 3) & 1) * 8;
    int ch = ks * 2 + (lane >> 4);
    ldmatrix_x4(qf[ks], sQ + swz<D>(r, ch));
  }

  float o_acc[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int pa = row0 + (lane >> 2), pb = pa + 8;
  const int pos_a = (pa < rows_total) ? ctx + pa / g : -1;
  const int pos_b = (pb < rows_total) ? ctx + pb / g : -1;
  const int lo_a = (p.window > 0) ? pos_a - p.window + 1 : 0;
  const int lo_b = (p.window > 0) ? pos_b - p.window + 1 : 0;

  for (int i = 0; i < my_tiles; ++i) {
    {
      int nxt = i + kStages - 1;
      if (nxt < my_tiles) load_tile(nxt, nxt % kStages);
      cp_async_commit();
    }
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const T* tK = my_kv + (i % kStages) * 2 * kTileElems;
    const T* tV = tK + kTileElems;

    // ---- S[16 x 16] = Q K^T : all K fragments first, then four independent MMA chains
    uint32_t kf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      int r = (lane & 7) + (lane >> 4) * 8;
      int ch = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(kf[ks], tK + swz<D>(r, ch));
    }
    float s0[2][4], s1[2][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) { s0[0][e] = s0[1][e] = s1[0][e] = s1[1][e] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ks += 2) {
      MT::mma(s0[0], qf[ks], kf[ks][0], kf[ks][1]);
      MT::mma(s1[0], qf[ks], kf[ks][2], kf[ks][3]);
      MT::mma(s0[1], qf[ks + 1], kf[ks + 1][0], kf[ks + 1][1]);
      MT::mma(s1[1], qf[ks + 1], kf[ks + 1][2], kf[ks + 1][3]);
    }
    float sc[2][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) { sc[0][e] = s0[0][e] + s0[1][e]; sc[1][e] = s1[0][e] + s1[1][e]; }

    // ---- mask + online softmax (base 2)
    const int key0 = kv_begin + (tile_lo + warp + i * kWarps) * kDecTile + (lane & 3) * 2;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        int key = key0 + n * 8 + e;
        bool in = key < kv_end;
        float va = (in && key <= pos_a && key >= lo_a) ? sc[n][e] * p.scale_log2 : -INFINITY;
        float vb = (in && key <= pos_b && key >= lo_b) ? sc[n][2 + e] * p.scale_log2 : -INFINITY;
        sc[n][e] = va;
        sc[n][2 + e] = vb;
        mx_a = fmaxf(mx_a, va);
        mx_b = fmaxf(mx_b, vb);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 2));
    const float mn_a = fmaxf(m_run[0], mx_a), mn_b = fmaxf(m_run[1], mx_b);
    const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    const float corr_a = exp2f(m_run[0] - ms_a), corr_b = exp2f(m_run[1] - ms_b);
    m_run[0] = mn_a;
    m_run[1] = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float pa_ = exp2f(sc[n][e] - ms_a), pb_ = exp2f(sc[n][2 + e] - ms_b);
        sc[n][e] = pa_;
        sc[n][2 + e] = pb_;
        sum_a += pa_;
        sum_b += pb_;
      }
    }
    l_run[0] = l_run[0] * corr_a + sum_a;
    l_run[1] = l_run[1] * corr_b + sum_b;
    if (__any_sync(0xffffffff, corr_a != 1.f || corr_b != 1.f)) {
#pragma unroll
      for (int d = 0; d < DT; ++d) {
        o_acc[d][0] *= corr_a; o_acc[d][1] *= corr_a;
        o_acc[d][2] *= corr_b; o_acc[d][3] *= corr_b;
      }
    }
    // ---- O += P V : 16 keys = one k-step; every d-tile has its own accumulator
    uint32_t a[4];
    a[0] = MT::pack(sc[0][0], sc[0][1]);
    a[1] = MT::pack(sc[0][2], sc[0][3]);
    a[2] = MT::pack(sc[1][0], sc[1][1]);
    a[3] = MT::pack(sc[1][2], sc[1][3]);
#pragma unroll
    for (int dp = 0; dp < DT / 2; dp += 2) {
      uint32_t b0[4], b1[4];
      int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4_trans(b0, tV + swz<D>(r, dp * 2 + (lane >> 4)));
      ldmatrix_x4_trans(b1, tV + swz<D>(r, (dp + 1) * 2 + (lane >> 4)));
      MT::mma(o_acc[2 * dp], a, b0[0], b0[1]);
      MT::mma(o_acc[2 * dp + 1], a, b0[2], b0[3]);
      MT::mma(o_acc[2 * dp + 2], a, b1[0], b1[1]);
      MT::mma(o_acc[2 * dp + 3], a, b1[2], b1[3]);
    }
    __syncwarp();  // the stage is refilled by this warp's next prefetch
  }
  cp_async_wait<0>();

  l_run[0] += __shfl_xor_sync(0xffffffff, l_run[0], 1);
  l_run[0] += __shfl_xor_sync(0xffffffff, l_run[0], 2);
  l_run[1] += __shfl_xor_sync(0xffffffff, l_run[1], 1);
  l_run[1] += __shfl_xor_sync(0xffffffff, l_run[1], 2);

  // ---------------------------------------------------------------- merge the warps' states
  __syncthreads();
  float* sO = reinterpret_cast<float*>(sKV);  // [kWarps][16][D]
  float* sM = sO + kWarps * 16 * D;           // [kWarps][16]
  float* sL = sM + kWarps * 16;               // [kWarps][16]
  {
    int ra = lane >> 2, rb = ra + 8;
    if ((lane & 3) == 0) {
      sM[warp * 16 + ra] = m_run[0]; sM[warp * 16 + rb] = m_run[1];
      sL[warp * 16 + ra] = l_run[0]; sL[warp * 16 + rb] = l_run[1];
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      int col = d * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(&sO[(warp * 16 + ra) * D + col]) = make_float2(o_acc[d][0], o_acc[d][1]);
      *reinterpret_cast<float2*>(&sO[(warp * 16 + rb) * D + col]) = make_float2(o_acc[d][2], o_acc[d][3]);
    }
  }
  __syncthreads();
  // thread -> (row, 2 adjacent columns): consecutive threads write consecutive output words
  constexpr int kPairs = D / 2;
  for (int idx = tid; idx < 16 * kPairs; idx += kWarps * 32) {
    const int r = idx / kPairs, c = (idx % kPairs) * 2;
    const int prow = row0 + r;
    if (prow >= rows_total) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sM[w * 16 + r]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, ax = 0.f, ay = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      float wg = exp2f(sM[w * 16 + r] - Ms);
      L += sL[w * 16 + r] * wg;
      float2 v = *reinterpret_cast<const float2*>(&sO[(w * 16 + r) * D + c]);
      ax += v.x * wg;
      ay += v.y * wg;
    }
    const int tok = prow / g, hh = kvh * g + prow % g;
    const int64_t orow = (int64_t)(qs + tok) * p.Hq + hh;
    if (p.num_splits == 1) {
      float den = L;
      if (p.sinks != nullptr) den += exp2f(p.sinks[hh] * 1.4426950408889634f - Ms);
      const float inv = den > 0.f ? 1.f / den : 0.f;
      *reinterpret_cast<uint32_t*>(reinterpret_cast<T*>(p.out) + orow * D + c) = MT::pack(ax * inv, ay * inv);
    } else {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      *reinterpret_cast<float2*>(p.ws_o + ((int64_t)split * p.T * p.Hq + orow) * D + c) = make_float2(ax * inv, ay * inv);
      if (c == 0) p.ws_lse[(int64_t)split * p.T * p.Hq + orow] = (L > 0.f) ? Ms + log2f(L) : -INFINITY;
    }
  }
  if (p.num_splits == 1 || !p.fuse_merge) return;
  // ---------------------------------------------------------------- split-KV merge by the last CTA to arrive
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  const int ticket_idx = (req * p.Hkv + kvh) * gridDim.x + blockIdx.x;
  if (tid == 0) s_last = (atomicAdd(&g_decode_tickets[ticket_idx], 1) == p.num_splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = tid; idx < 16 * kPairs; idx += kWarps * 32) {
    const int r = idx / kPairs, c = (idx % kPairs) * 2;
    const int prow = row0 + r;
    if (prow >= rows_total) continue;
    const int tok = prow / g, hh = kvh * g + prow % g;
    const int64_t orow = (int64_t)(qs + tok) * p.Hq + hh;
    const int64_t sstride = p.T * p.Hq;
    float M = -INFINITY;
    for (int s2 = 0; s2 < p.num_splits; ++s2) M = fmaxf(M, __ldcg(p.ws_lse + s2 * sstride + orow));
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float den = 0.f, ax = 0.f, ay = 0.f;
    for (int s2 = 0; s2 < p.num_splits; ++s2) {
      const float wg = exp2f(__ldcg(p.ws_lse + s2 * sstride + orow) - Ms);
      den += wg;
      if (wg > 0.f) {
        float2 v = __ldcg(reinterpret_cast<const float2*>(p.ws_o + (s2 * sstride + orow) * D + c));
        ax += v.x * wg;
        ay += v.y * wg;
      }
    }
    if (p.sinks != nullptr) den += exp2f(p.sinks[hh] * 1.4426950408889634f - Ms);
    const float inv = den > 0.f ? 1.f / den : 0.f;
    *reinterpret_cast<uint32_t*>(reinterpret_cast<T*>(p.out) + orow * D + c) = MT::pack(ax * inv, ay * inv);
  }
  if (tid == 0) g_decode_tickets[ticket_idx] = 0;
}

template <typename T, int D, int kWarps, int kStages>
static int launch_decode(AttnParams p, int B, int max_q_rows, cudaStream_t st, bool* merged) {
  size_t kv_bytes = (size_t)kWarps * kStages * 2 * kDecTile * D * sizeof(T);
  size_t merge_bytes = (size_t)(kWarps * 16 * D + 2 * kWarps * 16) * sizeof(float);
  size_t smem = (size_t)16 * D * sizeof(T) + (kv_bytes > merge_bytes ? kv_bytes : merge_bytes);
  auto kern = paged_decode_kernel<T, D, kWarps, kStages>;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_q_rows + 15) / 16, p.Hkv, B * p.num_splits);
  static const bool fuse_on = [] { const char* e = getenv("B200_ATTN_FUSE_MERGE"); return !(e != nullptr && e[0] == '0'); }();
  p.fuse_merge = fuse_on && p.num_splits > 1 && (int64_t)B * p.Hkv * grid.x <= kMaxTickets;
  *merged = p.fuse_merge != 0;
  return (int)launch_pdl(kern, grid, dim3(kWarps * 32), smem, st, p);
}

int paged_decode_dispatch(const AttnParams& p, int B, int max_q_rows, int D, int dtype, cudaStream_t st, bool* merged) {
  *merged = false;
  if (p.block_size % kDecTile) return 4;
  if (dtype == kBF16) {
    if (D == 128) return launch_decode<__nv_bfloat16, 128, 4, 3>(p, B, max_q_rows, st, merged);
    if (D == 64) return launch_decode<__nv_bfloat16, 64, 4, 4>(p, B, max_q_rows, st, merged);
    if (D == 256) return launch_decode<__nv_bfloat16, 256, 4, 2>(p, B, max_q_rows, st, merged);
  } else if (dtype == kF16) {
    if (D == 128) return launch_decode<__half, 128, 4, 3>(p, B, max_q_rows, st, merged);
    if (D == 64) return launch_decode<__half, 64, 4, 4>(p, B, max_q_rows, st, merged);
    if (D == 256) return launch_decode<__half, 256, 4, 2>(p, B, max_q_rows, st, merged);
  }
  return 3;
}

}  // namespace b200
