// Weight-absorbed MLA attention over the latent cache (dense paged or sparse by index list).
//
//   q   [T, N, 576]   = [q_nope . W_UK (512) | q_pe (64)]
//   kv  [slots, 576]  = [kv_c (512) | k_pe (64)]  (paged: slot = block * block_size + offset)
//   out [T, N, 512]   = softmax(q . kv^T * scale) . kv[:, :512]
//
// One CTA = 4 warps serves (query token, tile of 16 heads, kv split): all heads of a token share
// one latent "KV head", so the 16 heads are the M side of the MMAs.  Keys come either from the
// request's block table (positions 0..pos of the token, causal) or from the token's own index list
// (DeepSeek sparse attention, -1 = unused entry).  Per 32-key tile: warp w computes S for keys
// [8w, 8w+8) (36 k-steps of m16n8k16), the row maxima are exchanged through shared memory, P goes
// to shared memory in bf16 and warp w accumulates output dims [128w, 128w+128) (V is the first 512
// dims of the same shared-memory tile, so the latent row is read from HBM once).
// Split partials (fp32 O, log2-sum-exp) are merged by merge_splits_kernel.
#include "../api.h"
#include "../common/launch.cuh"
#include "attn_common.cuh"

namespace b200 {

constexpr int kMlaD = 576;
constexpr int kMlaV = 512;
constexpr int kMlaTile = 32;
constexpr int kMlaStages = 2;
constexpr int kMlaThreads = 128;

struct MlaParams {
  const void* q;            // [T, N, 576]
  const void* kv;           // flat [slots, 576]
  void* out;                // [T, N, 512]
  float* ws_o;              // [splits, T, N, 512]
  float* ws_lse;            // [splits, T, N]
  const int* block_tables;  // dense: [B, max_blocks]
  const int* seq_lens;      // dense: [B]
  const int* qsl;           // dense: [B + 1]
  const int* req_of_token;  // dense: [T]
  const int* indices;       // sparse: [T, topk] global slots, -1 = none
  int N, block_size, max_blocks, num_splits, topk, B;
  int64_t total_slots, T;
  float scale_log2;
};

template <typename T, bool kSparse>
__global__ void __launch_bounds__(kMlaThreads) mla_attention_kernel(MlaParams p) {
  constexpr int D = kMlaD;
  constexpr int CH = D / 8;  // 72 chunks of 16 bytes per row
  using MT = MmaTraits<T>;
  extern __shared__ __align__(16) uint8_t smem_mla[];
  T* sQ = reinterpret_cast<T*>(smem_mla);                 // [16][576]
  T* sKV = sQ + 16 * D;                                   // [stages][32][576]
  T* sP = sKV + kMlaStages * kMlaTile * D;                // [2][16][32]  (tile parity)
  float* sMax = reinterpret_cast<float*>(sP + 2 * 16 * kMlaTile);  // [2][4][16]
  float* sSum = sMax + 2 * 4 * 16;                        // [4][16]
  int* sSlot = reinterpret_cast<int*>(sSum + 4 * 16);     // [stages][32] resolved slot per key row

  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t t = blockIdx.y;
  const int head0 = blockIdx.x * 16;
  const int split = blockIdx.z;
  int n_keys;       // keys this token may attend (dense: pos + 1, sparse: topk entries)
  const int* bt = nullptr;
  if (kSparse) {
    n_keys = p.topk;
  } else {
    const int req = p.req_of_token[t];
    if (req < 0 || req >= p.B) return;
    const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
    const int seq_len = p.seq_lens[req];
    n_keys = seq_len - q_len + (int)(t - qs) + 1;
    bt = p.block_tables + (int64_t)req * p.max_blocks;
  }
  const int tiles_all = (max(n_keys, 0) + kMlaTile - 1) / kMlaTile;
  const int per_split = (tiles_all + p.num_splits - 1) / p.num_splits;
  const int tile_lo = split * per_split;
  const int tile_hi = min(tiles_all, tile_lo + per_split);
  const int n_tiles = max(0, tile_hi - tile_lo);

  const T* q_base = reinterpret_cast<const T*>(p.q) + (t * p.N + head0) * (int64_t)D;
  const T* kv_base = reinterpret_cast<const T*>(p.kv);

  for (int c = tid; c < 16 * CH; c += kMlaThreads) {
    int r = c / CH, ch = c % CH;
    bool valid = head0 + r < p.N;
    cp_async16(sQ + swz<D>(r, ch), q_base + (valid ? (int64_t)r * D + ch * 8 : 0), valid);
  }
  cp_async_commit();

  auto load_tile = [&](int i, int stage) {
    const int base = (tile_lo + i) * kMlaTile;
    // resolve the 32 key slots once (first warp), then all threads copy
    if (tid < kMlaTile) {
      int j = base + tid;
      int64_t slot = -1;
      if (j < n_keys) {
        if (kSparse) {
          slot = p.indices[t * p.topk + j];
        } else {
          int bi = j / p.block_size;
          int64_t blk = (bi < p.max_blocks) ? bt[bi] : -1;
          slot = blk >= 0 ? blk * p.block_size + j % p.block_size : -1;
        }
        if (slot >= p.total_slots) slot = -1;
      }
      sSlot[stage * kMlaTile + tid] = (int)slot;
    }
    __syncthreads();
    T* dst = sKV + stage * kMlaTile * D;
    for (int c = tid; c < kMlaTile * CH; c += kMlaThreads) {
      int r = c / CH, ch = c % CH;
      int slot = sSlot[stage * kMlaTile + r];
      bool valid = slot >= 0;
      cp_async16(dst + swz<D>(r, ch), kv_base + (valid ? (int64_t)slot * D + ch * 8 : 0), valid);
    }
  };

  if (n_tiles > 0) load_tile(0, 0);
  cp_async_commit();

  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_part[2] = {0.f, 0.f};  // this warp's keys only

  for (int i = 0; i < n_tiles; ++i) {
    const int stage = i & 1;
    if (i + 1 < n_tiles) load_tile(i + 1, stage ^ 1);  // (contains a __syncthreads)
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* tK = sKV + stage * kMlaTile * D;
    const int par = i & 1;

    // ---- S[16 heads x 8 keys] for this warp's keys
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    float s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t a0[4], a1[4], b[4];
      int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(a0, sQ + swz<D>(r, ks * 2 + (lane >> 4)));
      ldmatrix_x4(a1, sQ + swz<D>(r, (ks + 1) * 2 + (lane >> 4)));
      // keys warp*8 .. +8 ; x4 = (k-step ks lo, ks hi, ks+1 lo, ks+1 hi)
      int kr = warp * 8 + (lane & 7);
      ldmatrix_x4(b, tK + swz<D>(kr, ks * 2 + (lane >> 3)));
      MT::mma(s, a0, b[0], b[1]);
      MT::mma(s2, a1, b[2], b[3]);
    }
    // rows: a = lane/4, b = a + 8 ; cols (keys): (lane%4)*2 + {0,1}
    const int key0 = (tile_lo + i) * kMlaTile + warp * 8 + (lane & 3) * 2;
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int key = key0 + (e & 1);
      bool ok = key < n_keys && sSlot[stage * kMlaTile + warp * 8 + (lane & 3) * 2 + (e & 1)] >= 0;
      v[e] = ok ? (s[e] + s2[e]) * p.scale_log2 : -INFINITY;
    }
    float mx_a = fmaxf(v[0], v[1]), mx_b = fmaxf(v[2], v[3]);
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffff, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffff, mx_b, 2));
    if ((lane & 3) == 0) {
      sMax[(par * 4 + warp) * 16 + (lane >> 2)] = mx_a;
      sMax[(par * 4 + warp) * 16 + (lane >> 2) + 8] = mx_b;
    }
    __syncthreads();
    float tm_a = -INFINITY, tm_b = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      tm_a = fmaxf(tm_a, sMax[(par * 4 + w) * 16 + (lane >> 2)]);
      tm_b = fmaxf(tm_b, sMax[(par * 4 + w) * 16 + (lane >> 2) + 8]);
    }
    const float mn_a = fmaxf(m_run[0], tm_a), mn_b = fmaxf(m_run[1], tm_b);
    const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    const float corr_a = exp2f(m_run[0] - ms_a), corr_b = exp2f(m_run[1] - ms_b);
    m_run[0] = mn_a;
    m_run[1] = mn_b;
    const float p0 = exp2f(v[0] - ms_a), p1 = exp2f(v[1] - ms_a), p2 = exp2f(v[2] - ms_b), p3 = exp2f(v[3] - ms_b);
    l_part[0] = l_part[0] * corr_a + p0 + p1;
    l_part[1] = l_part[1] * corr_b + p2 + p3;
    {
      T* dP = sP + par * 16 * kMlaTile;
      int col = warp * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(dP + (lane >> 2) * kMlaTile + col) = MT::pack(p0, p1);
      *reinterpret_cast<uint32_t*>(dP + ((lane >> 2) + 8) * kMlaTile + col) = MT::pack(p2, p3);
    }
#pragma unroll
    for (int d = 0; d < 16; ++d) {
      o_acc[d][0] *= corr_a; o_acc[d][1] *= corr_a;
      o_acc[d][2] *= corr_b; o_acc[d][3] *= corr_b;
    }
    __syncthreads();
    // ---- O[16 x 128 (dims 128w..)] += P[16 x 32] . V[32 x 128]
    const T* tP = sP + par * 16 * kMlaTile;
#pragma unroll
    for (int kt = 0; kt < kMlaTile / 16; ++kt) {
      uint32_t a[4];
      {
        // P tile is small and unswizzled: [16][32] bf16, row stride 64 bytes
        int r = (lane & 7) + ((lane >> 3) & 1) * 8;
        int cb = kt * 16 + (lane >> 4) * 8;
        ldmatrix_x4(a, tP + r * kMlaTile + cb);
      }
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b[4];
        int r = kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        int ch = warp * 16 + dp * 2 + (lane >> 4);
        ldmatrix_x4_trans(b, tK + swz<D>(r, ch));
        MT::mma(o_acc[2 * dp], a, b[0], b[1]);
        MT::mma(o_acc[2 * dp + 1], a, b[2], b[3]);
      }
    }
    // the next iteration's load_tile starts with a __syncthreads before touching this stage's twin
  }
  cp_async_wait<0>();

  // ---- total row sums over the four warps
  l_part[0] += __shfl_xor_sync(0xffffffff, l_part[0], 1);
  l_part[0] += __shfl_xor_sync(0xffffffff, l_part[0], 2);
  l_part[1] += __shfl_xor_sync(0xffffffff, l_part[1], 1);
  l_part[1] += __shfl_xor_sync(0xffffffff, l_part[1], 2);
  __syncthreads();
  if ((lane & 3) == 0) {
    sSum[warp * 16 + (lane >> 2)] = l_part[0];
    sSum[warp * 16 + (lane >> 2) + 8] = l_part[1];
  }
  __syncthreads();
  float l_a = 0.f, l_b = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) { l_a += sSum[w * 16 + (lane >> 2)]; l_b += sSum[w * 16 + (lane >> 2) + 8]; }

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = (lane >> 2) + half * 8;
    if (head0 + row >= p.N) continue;
    const float l = half ? l_b : l_a;
    const float m = m_run[half];
    const float ms = (m == -INFINITY) ? 0.f : m;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int64_t orow = t * p.N + head0 + row;
    if (p.num_splits == 1) {
      T* dst = reinterpret_cast<T*>(p.out) + orow * kMlaV + warp * 128;
#pragma unroll
      for (int d = 0; d < 16; ++d) {
        int col = d * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(dst + col) = MT::pack(o_acc[d][half * 2] * inv, o_acc[d][half * 2 + 1] * inv);
      }
    } else {
      float* dst = p.ws_o + ((int64_t)split * p.T * p.N + orow) * kMlaV + warp * 128;
#pragma unroll
      for (int d = 0; d < 16; ++d) {
        int col = d * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[d][half * 2] * inv, o_acc[d][half * 2 + 1] * inv);
      }
      if (warp == 0 && (lane & 3) == 0)
        p.ws_lse[(int64_t)split * p.T * p.N + orow] = (l > 0.f) ? ms + log2f(l) : -INFINITY;
    }
  }
}

template <typename T, bool kSparse>
static int launch_mla(const MlaParams& p, cudaStream_t st) {
  size_t smem = (size_t)(16 * kMlaD + kMlaStages * kMlaTile * kMlaD + 2 * 16 * kMlaTile) * sizeof(T) +
                (2 * 4 * 16 + 4 * 16) * sizeof(float) + kMlaStages * kMlaTile * sizeof(int);
  auto kern = mla_attention_kernel<T, kSparse>;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((p.N + 15) / 16, (unsigned)p.T, p.num_splits);
  return (int)launch_pdl(kern, grid, dim3(kMlaThreads), smem, st, p);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_mla_attention(void* out, const void* q, const void* kv, const int* block_tables,
                                  const int* seq_lens, const int* qsl, const int* req_of_token, const int* indices,
                                  float* ws_o, float* ws_lse, int64_t T_, int B, int N, int block_size, int max_blocks,
                                  int64_t total_slots, int topk, int num_splits, float scale, int dtype,
                                  cudaStream_t st) {
  if (T_ == 0) return 0;
  MlaParams p;
  p.q = q; p.kv = kv; p.out = out; p.ws_o = ws_o; p.ws_lse = ws_lse; p.block_tables = block_tables;
  p.seq_lens = seq_lens; p.qsl = qsl; p.req_of_token = req_of_token; p.indices = indices;
  p.N = N; p.block_size = block_size; p.max_blocks = max_blocks; p.num_splits = num_splits; p.topk = topk; p.B = B;
  p.total_slots = total_slots; p.T = T_;
  p.scale_log2 = scale * 1.4426950408889634f;
  const bool sparse = indices != nullptr;
  if (!sparse && block_size % kMlaTile) return 4;
  int rc;
  if (dtype == kBF16) rc = sparse ? launch_mla<__nv_bfloat16, true>(p, st) : launch_mla<__nv_bfloat16, false>(p, st);
  else if (dtype == kF16) rc = sparse ? launch_mla<__half, true>(p, st) : launch_mla<__half, false>(p, st);
  else return 1;
  if (rc != 0 || num_splits == 1) return rc;
  return b200_merge_splits(out, ws_o, ws_lse, T_ * N, N, kMlaV, num_splits, T_, dtype, st);
}
