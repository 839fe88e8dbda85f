// Unified varlen paged GQA attention (prefill with cached prefix, decode, speculative verify).
//
// One CTA = 4 warps handles one (request, kv head, q tile, kv split).  The queries of a GQA group
// are packed along M: packed row p -> (token p / g, head p % g), so a decode step of a 4:1 group
// still feeds full 16-row MMA tiles.  Two warp layouts:
//   WM=4, WN=1  prefill: 64 packed rows, every warp sees all 64 keys of a KV tile
//   WM=1, WN=4  decode : 16 packed rows, warp w owns keys [16w, 16w+16) of every KV tile and keeps
//                        its own online-softmax state; the four states are merged at the end
// K/V tiles (64 keys) are gathered from the paged cache with 16-byte cp.async into XOR-swizzled
// shared memory, multi-stage.  Split-KV partials (fp32 O and log2-sum-exp) go to a workspace and
// are combined by merge_splits_kernel.  The math core is mma.sync m16n8k16 (bf16/fp16, fp32
// accumulate); the decode path is bandwidth-bound by the KV read.
//
// Block-table entries and derived addresses are range-checked; out-of-range keys read as zeros
// and are masked.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "attn_common.cuh"

namespace b200 {

template <typename T, int D, int WM, int WN, int kStages>
__global__ void __launch_bounds__(kAttnThreads) paged_attention_kernel(AttnParams p) {
  constexpr int BM = 16 * WM;          // packed query rows per CTA
  constexpr int NW = kTileN / WN;      // keys per warp per KV tile
  constexpr int NT = NW / 8;           // S n-tiles per warp
  constexpr int CH = D / 8;            // 16-byte chunks per row
  constexpr int DT = D / 8;            // O n-tiles
  using MT = MmaTraits<T>;
  extern __shared__ __align__(16) uint8_t smem_attn[];
  T* sQ = reinterpret_cast<T*>(smem_attn);           // [BM][D]
  T* sK = sQ + BM * D;                               // [kStages][64][D]
  T* sV = sK + kStages * kTileN * D;                 // [kStages][64][D]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp % WM, wn = warp / WM;
  const int g = p.Hq / p.Hkv;
  const int kvh = blockIdx.y;
  const int req = blockIdx.z / p.num_splits;
  const int split = blockIdx.z % p.num_splits;
  const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
  const int seq_len = p.seq_lens[req];
  const int rows_total = q_len * g;
  const int row0 = blockIdx.x * BM;
  if (row0 >= rows_total || q_len <= 0) return;
  const int ctx = seq_len - q_len;  // absolute position of this request's first query token
  const int tok_lo = row0 / g;
  const int tok_hi = min(q_len - 1, (row0 + BM - 1) / g);
  // keys visible to any row of this tile
  // window < 0 selects bidirectional attention (vision towers): every row sees the whole sequence
  const bool bidir = p.window < 0;
  int kv_end = bidir ? seq_len : min(seq_len, ctx + tok_hi + 1);
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, ctx + tok_lo - p.window + 1) / kTileN * kTileN;
  // this split's share (whole tiles)
  int n_tiles_all = (kv_end - kv_begin + kTileN - 1) / kTileN;
  int tiles_per_split = (n_tiles_all + p.num_splits - 1) / p.num_splits;
  int tile_lo = split * tiles_per_split;
  int tile_hi = min(n_tiles_all, tile_lo + tiles_per_split);
  const int n_tiles = max(0, tile_hi - tile_lo);
  const int kv0 = kv_begin + tile_lo * kTileN;

  const T* q_base = reinterpret_cast<const T*>(p.q);
  const T* kv_base = reinterpret_cast<const T*>(p.kv_cache);
  const int* bt = p.block_tables + (int64_t)req * p.max_blocks;

  // ---------------------------------------------------------------- loads
  auto load_q = [&]() {
    for (int c = tid; c < BM * CH; c += kAttnThreads) {
      int r = c / CH, ch = c % CH;
      int prow = row0 + r;
      bool valid = prow < rows_total;
      int tok = valid ? prow / g : 0, hh = valid ? prow % g : 0;
      const T* src = q_base + ((int64_t)(qs + tok) * p.Hq + kvh * g + hh) * D + ch * 8;
      cp_async16(sQ + swz<D>(r, ch), src, valid);
    }
  };
  auto load_kv = [&](int tile, int stage) {
    T* dK = sK + stage * kTileN * D;
    T* dV = sV + stage * kTileN * D;
    const int base = kv0 + tile * kTileN;
    for (int c = tid; c < kTileN * CH; c += kAttnThreads) {
      int r = c / CH, ch = c % CH;
      int j = base + r;
      bool valid = j < kv_end;
      int64_t blk = 0;
      if (valid) {
        int bi = j / p.block_size;
        blk = (bi < p.max_blocks) ? bt[bi] : -1;
        valid = blk >= 0 && blk < p.num_blocks;
        if (!valid) blk = 0;
      }
      int off = valid ? j % p.block_size : 0;
      const T* srcK = kv_base + ((((blk * 2 + 0) * p.Hkv + kvh) * p.block_size + off) * (int64_t)D) + ch * 8;
      const T* srcV = srcK + (int64_t)p.Hkv * p.block_size * D;
      cp_async16(dK + swz<D>(r, ch), srcK, valid);
      cp_async16(dV + swz<D>(r, ch), srcV, valid);
    }
  };

  load_q();
  cp_async_commit();
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) load_kv(s, s);
    cp_async_commit();
  }

  // ---------------------------------------------------------------- state
  float o_acc[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  // rows owned by this thread: r_a = wm*16 + lane/4, r_b = r_a + 8
  const int r_a = wm * 16 + (lane >> 2), r_b = r_a + 8;
  const int pa = row0 + r_a, pb = row0 + r_b;
  const int pos_a = (pa < rows_total) ? (bidir ? seq_len - 1 : ctx + pa / g) : -1;  // -1: padding row (sees nothing)
  const int pos_b = (pb < rows_total) ? (bidir ? seq_len - 1 : ctx + pb / g) : -1;
  const int lo_a = (p.window > 0) ? pos_a - p.window + 1 : 0;
  const int lo_b = (p.window > 0) ? pos_b - p.window + 1 : 0;

  for (int tile = 0; tile < n_tiles; ++tile) {
    // prefetch tile + kStages - 1
    {
      int nxt = tile + kStages - 1;
      if (nxt < n_tiles) load_kv(nxt, nxt % kStages);
      cp_async_commit();
    }
    cp_async_wait<kStages - 1>();
    __syncthreads();
    const T* tK = sK + (tile % kStages) * kTileN * D;
    const T* tV = sV + (tile % kStages) * kTileN * D;

    // ---- S = Q K^T  (this warp: rows wm*16..+16, keys wn*NW..+NW)
    float s_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      {
        int r = wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        int ch = ks * 2 + (lane >> 4);
        ldmatrix_x4(a, sQ + swz<D>(r, ch));
      }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b[4];
        int r = wn * NW + np * 16 + (lane & 7) + (lane >> 4) * 8;
        int ch = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b, tK + swz<D>(r, ch));
        MT::mma(s_acc[2 * np], a, b[0], b[1]);
        MT::mma(s_acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    // ---- mask + online softmax (base 2)
    const int key0 = kv0 + tile * kTileN + wn * NW + (lane & 3) * 2;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        int key = key0 + i * 8 + e;
        bool in = key < kv_end;
        float va = (in && key <= pos_a && key >= lo_a) ? s_acc[i][e] * p.scale_log2 : -INFINITY;
        float vb = (in && key <= pos_b && key >= lo_b) ? s_acc[i][2 + e] * p.scale_log2 : -INFINITY;
        s_acc[i][e] = va;
        s_acc[i][2 + e] = vb;
        mx_a = fmaxf(mx_a, va);
        mx_b = fmaxf(mx_b, vb);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 2));
    float mn_a = fmaxf(m_run[0], mx_a), mn_b = fmaxf(m_run[1], mx_b);
    float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    float corr_a = exp2f(m_run[0] - ms_a), corr_b = exp2f(m_run[1] - ms_b);  // exp2(-inf) = 0
    m_run[0] = mn_a;
    m_run[1] = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float pa_ = exp2f(s_acc[i][e] - ms_a), pb_ = exp2f(s_acc[i][2 + e] - ms_b);
        s_acc[i][e] = pa_;
        s_acc[i][2 + e] = pb_;
        sum_a += pa_;
        sum_b += pb_;
      }
    }
    l_run[0] = l_run[0] * corr_a + sum_a;
    l_run[1] = l_run[1] * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      o_acc[i][0] *= corr_a; o_acc[i][1] *= corr_a;
      o_acc[i][2] *= corr_b; o_acc[i][3] *= corr_b;
    }
    // ---- O += P V
#pragma unroll
    for (int kt = 0; kt < NW / 16; ++kt) {
      uint32_t a[4];
      a[0] = MT::pack(s_acc[2 * kt][0], s_acc[2 * kt][1]);
      a[1] = MT::pack(s_acc[2 * kt][2], s_acc[2 * kt][3]);
      a[2] = MT::pack(s_acc[2 * kt + 1][0], s_acc[2 * kt + 1][1]);
      a[3] = MT::pack(s_acc[2 * kt + 1][2], s_acc[2 * kt + 1][3]);
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        uint32_t b[4];
        int r = wn * NW + kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        int ch = dp * 2 + (lane >> 4);
        ldmatrix_x4_trans(b, tV + swz<D>(r, ch));
        MT::mma(o_acc[2 * dp], a, b[0], b[1]);
        MT::mma(o_acc[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // stage may be overwritten by the next prefetch
  }
  cp_async_wait<0>();

  // quad-reduce the row sums
  l_run[0] += __shfl_xor_sync(0xffffffff, l_run[0], 1);
  l_run[0] += __shfl_xor_sync(0xffffffff, l_run[0], 2);
  l_run[1] += __shfl_xor_sync(0xffffffff, l_run[1], 1);
  l_run[1] += __shfl_xor_sync(0xffffffff, l_run[1], 2);

  // ---------------------------------------------------------------- cross-warp merge (WN > 1)
  if (WN > 1) {
    __syncthreads();
    float* sO = reinterpret_cast<float*>(sK);          // [WN][16][D]
    float* sM = sO + WN * 16 * D;                      // [WN][16]
    float* sL = sM + WN * 16;                          // [WN][16]
    {
      int ra = lane >> 2, rb = ra + 8;
      if ((lane & 3) == 0) {
        sM[wn * 16 + ra] = m_run[0]; sM[wn * 16 + rb] = m_run[1];
        sL[wn * 16 + ra] = l_run[0]; sL[wn * 16 + rb] = l_run[1];
      }
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        int col = i * 8 + (lane & 3) * 2;
        sO[(wn * 16 + ra) * D + col] = o_acc[i][0];
        sO[(wn * 16 + ra) * D + col + 1] = o_acc[i][1];
        sO[(wn * 16 + rb) * D + col] = o_acc[i][2];
        sO[(wn * 16 + rb) * D + col + 1] = o_acc[i][3];
      }
    }
    __syncthreads();
    // thread -> (row = tid / 8, 16 columns strided by 8) : 128 threads cover 16 rows x 8 column groups
    int r = tid >> 3, cg = tid & 7;
    int prow = row0 + r;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WN; ++w) M = fmaxf(M, sM[w * 16 + r]);
    float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, wgt[WN];
#pragma unroll
    for (int w = 0; w < WN; ++w) { wgt[w] = exp2f(sM[w * 16 + r] - Ms); L += sL[w * 16 + r] * wgt[w]; }
    if (prow < rows_total) {
      int tok = prow / g, hh = kvh * g + prow % g;
      int64_t orow = (int64_t)(qs + tok) * p.Hq + hh;
      if (p.num_splits == 1) {
        float den = L;
        if (p.sinks != nullptr) den += exp2f(p.sinks[hh] * 1.4426950408889634f - Ms);
        float inv = den > 0.f ? 1.f / den : 0.f;
        T* dst = reinterpret_cast<T*>(p.out) + orow * D;
        for (int c = cg; c < D; c += 8) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < WN; ++w) acc += sO[(w * 16 + r) * D + c] * wgt[w];
          dst[c] = from_f<T>(acc * inv);
        }
      } else {
        float inv = L > 0.f ? 1.f / L : 0.f;
        float* dst = p.ws_o + ((int64_t)split * p.T * p.Hq + orow) * D;
        for (int c = cg; c < D; c += 8) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < WN; ++w) acc += sO[(w * 16 + r) * D + c] * wgt[w];
          dst[c] = acc * inv;
        }
        if (cg == 0) p.ws_lse[(int64_t)split * p.T * p.Hq + orow] = (L > 0.f) ? Ms + log2f(L) : -INFINITY;
      }
    }
    return;
  }

  // ---------------------------------------------------------------- direct epilogue (WN == 1)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    int prow = half ? pb : pa;
    if (prow >= rows_total) continue;
    int tok = prow / g, hh = kvh * g + prow % g;
    int64_t orow = (int64_t)(qs + tok) * p.Hq + hh;
    float m = m_run[half], l = l_run[half];
    float ms = (m == -INFINITY) ? 0.f : m;
    if (p.num_splits == 1) {
      float den = l;
      if (p.sinks != nullptr) den += exp2f(p.sinks[hh] * 1.4426950408889634f - ms);
      float inv = den > 0.f ? 1.f / den : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + orow * D;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        int col = i * 8 + (lane & 3) * 2;
        uint32_t v = MT::pack(o_acc[i][half * 2] * inv, o_acc[i][half * 2 + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + col) = v;
      }
    } else {
      float inv = l > 0.f ? 1.f / l : 0.f;
      float* dst = p.ws_o + ((int64_t)split * p.T * p.Hq + orow) * D;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        int col = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[i][half * 2] * inv, o_acc[i][half * 2 + 1] * inv);
      }
      if ((lane & 3) == 0) p.ws_lse[(int64_t)split * p.T * p.Hq + orow] = (l > 0.f) ? ms + log2f(l) : -INFINITY;
    }
  }
}

// Combine split-KV partials: out = sum_s w_s O_s / (sum_s w_s [+ sink]),  w_s = 2^(lse_s - max).
// One warp per (token, head) row.  Rows of padded requests (never written) are skipped via qsl.
template <typename T>
__global__ void merge_splits_kernel(T* __restrict__ out, float* __restrict__ lse_out, const float* __restrict__ ws_o,
                                    const float* __restrict__ ws_lse, const float* __restrict__ sinks, int64_t rows,
                                    int Hq, int D, int splits, int64_t T_, const int* __restrict__ qsl, int B) {
  griddep_launch();
  griddep_wait();
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int lane = threadIdx.x & 31;
  if (qsl != nullptr && row / Hq >= qsl[B]) return;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ws_lse[(int64_t)s * T_ * Hq + row]);
  float Ms = (M == -INFINITY) ? 0.f : M;
  float den = 0.f;
  for (int s = 0; s < splits; ++s) den += exp2f(ws_lse[(int64_t)s * T_ * Hq + row] - Ms);
  float den_o = den;
  if (sinks != nullptr) den_o += exp2f(sinks[row % Hq] * 1.4426950408889634f - Ms);
  float inv = den_o > 0.f ? 1.f / den_o : 0.f;
  for (int c = lane; c < D; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      float w = exp2f(ws_lse[(int64_t)s * T_ * Hq + row] - Ms);
      if (w > 0.f) acc += ws_o[((int64_t)s * T_ * Hq + row) * D + c] * w;
    }
    out[row * D + c] = from_f<T>(acc * inv);
  }
  if (lane == 0 && lse_out != nullptr) lse_out[row] = (den > 0.f) ? (Ms + log2f(den)) * 0.6931471805599453f : -INFINITY;
}

template <typename T, int D, int WM, int WN, int kStages>
static int launch_attn(const AttnParams& p, int B, int max_q_rows, cudaStream_t st) {
  constexpr int BM = 16 * WM;
  size_t kv_bytes = (size_t)kStages * 2 * kTileN * D * sizeof(T);
  size_t merge_bytes = (WN > 1) ? (size_t)(WN * 16 * D + 2 * WN * 16) * sizeof(float) : 0;
  size_t tail = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
  size_t smem = (size_t)BM * D * sizeof(T) + tail;
  auto kern = paged_attention_kernel<T, D, WM, WN, kStages>;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_q_rows + BM - 1) / BM, p.Hkv, B * p.num_splits);
  kern<<<grid, kAttnThreads, smem, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_paged_attention(void* out, const void* q, const void* kv_cache, const int* block_tables,
                                    const int* seq_lens, const int* qsl, const float* sinks, float* ws_o,
                                    float* ws_lse, int64_t T_, int B, int Hq, int Hkv, int D, int block_size,
                                    int max_blocks, int64_t num_blocks, int max_query_len, int num_splits,
                                    int window, float scale, int decode_layout, int dtype, cudaStream_t st) {
  if (B == 0 || T_ == 0) return 0;
  if (Hq % Hkv) return 2;
  AttnParams p;
  p.q = q; p.kv_cache = kv_cache; p.out = out; p.ws_o = ws_o; p.ws_lse = ws_lse;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.qsl = qsl; p.sinks = sinks;
  p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size; p.max_blocks = max_blocks; p.num_splits = num_splits;
  p.window = window; p.num_blocks = num_blocks; p.T = T_;
  p.scale_log2 = scale * 1.4426950408889634f;
  int max_q_rows = max_query_len * (Hq / Hkv);
  int rc = 3;
  bool merged = false;
  p.fuse_merge = 0;
  if (decode_layout && max_q_rows <= 16 && block_size % 16 == 0) {
    rc = paged_decode_dispatch(p, B, max_q_rows, D, dtype, st, &merged);
  } else {
#define B200_ATTN_CASE(TT, DD) rc = launch_attn<TT, DD, 4, 1, 2>(p, B, max_q_rows, st)
    if (dtype == kBF16) {
      if (D == 128) B200_ATTN_CASE(__nv_bfloat16, 128);
      else if (D == 64) B200_ATTN_CASE(__nv_bfloat16, 64);
      else if (D == 256) B200_ATTN_CASE(__nv_bfloat16, 256);
    } else if (dtype == kF16) {
      if (D == 128) B200_ATTN_CASE(__half, 128);
      else if (D == 64) B200_ATTN_CASE(__half, 64);
      else if (D == 256) B200_ATTN_CASE(__half, 256);
    }
#undef B200_ATTN_CASE
  }
  if (rc != 0) return rc;
  if (num_splits > 1 && !merged) {
    int64_t rows = T_ * Hq;
    if (dtype == kBF16)
      launch_pdl(merge_splits_kernel<__nv_bfloat16>, dim3((rows + 7) / 8), dim3(256), 0, st, (__nv_bfloat16*)out,
                 (float*)nullptr, (const float*)ws_o, (const float*)ws_lse, sinks, rows, Hq, D, num_splits, T_, qsl, B);
    else
      launch_pdl(merge_splits_kernel<__half>, dim3((rows + 7) / 8), dim3(256), 0, st, (__half*)out, (float*)nullptr,
                 (const float*)ws_o, (const float*)ws_lse, sinks, rows, Hq, D, num_splits, T_, qsl, B);
    return (int)cudaGetLastError();
  }
  return 0;
}

// Split-KV merge as a stand-alone entry (also used by the MLA kernels): rows = T * heads.
extern "C" int b200_merge_splits(void* out, const float* ws_o, const float* ws_lse, int64_t rows, int Hq, int D,
                                 int splits, int64_t T_, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (dtype == kBF16)
    return (int)launch_pdl(merge_splits_kernel<__nv_bfloat16>, dim3((rows + 7) / 8), dim3(256), 0, st,
                           (__nv_bfloat16*)out, (float*)nullptr, ws_o, ws_lse, (const float*)nullptr, rows, Hq, D,
                           splits, T_, (const int*)nullptr, 0);
  if (dtype == kF16)
    return (int)launch_pdl(merge_splits_kernel<__half>, dim3((rows + 7) / 8), dim3(256), 0, st, (__half*)out,
                           (float*)nullptr, ws_o, ws_lse, (const float*)nullptr, rows, Hq, D, splits, T_,
                           (const int*)nullptr, 0);
  return 1;
}
