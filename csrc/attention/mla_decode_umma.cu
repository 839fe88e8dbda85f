// Weight-absorbed MLA decode attention over the paged latent cache on tcgen05 + TMEM, fed by TMA.
//
//   q   [T, N, 576]        = [q_nope . W_UK (512) | q_pe (64)], a few query tokens per request (decode / MTP verify)
//   kv  [blocks, 64, 576]  = [kv_c (512) | k_pe (64)] per cached token, 16-bit
//   out [T, N, 512]        = softmax(q . kv^T * scale) . kv[:, :512]
//
// All heads of a token share ONE latent row, so a request's (heads x query tokens) rows are the small side of both
// products and the cached tokens the large one.  As in decode_umma.cu the operands are swapped so that the tensor
// core rows are full:
//     S^T[64 keys, R rows]   = K_page[64 keys, 576] . Q^T                         (36 k-steps, UMMA M = 64)
//     O^T[512 dims, R rows] += V_page^T[512 dims, 64 keys] . P[64 keys, R rows]    (4 M-tiles of 128 dims x 4 k-steps)
// with V = the first 512 dims of the SAME shared-memory page (MN-major operand), so a latent row crosses HBM once
// per CTA, whatever the number of heads or query tokens: a q_len = 2 verify step reads the cache once.
// TMEM: two S^T buffers (R columns each, lanes (i / 16) * 32 + i % 16 hold key i of an M = 64 accumulator) and four
// O^T tiles (R columns each): 6 R <= 192 columns.
//
// One CTA = (request, group of up to R / q_len heads, kv split).  192 threads: warp 0 TMA producer (one cache page =
// nine 64 x 64 boxes, 128-byte swizzle, 2-stage ring; pages of the old context are fetched before the
// programmatic-dependency wait when the caller vouches for the metadata), warp 1 MMA issuer, warps 2-5 softmax
// (thread = key) and epilogue (thread = output dim).  Lazy running maximum as in decode_umma.cu.  Split partials go
// through the fp32 workspace; the last CTA of a (request, head group) to arrive merges them.
// Every wait is bounded; on time-out the status word is set and the CTA unwinds.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/gemm_common.cuh"
#include "attn_common.cuh"

namespace b200 {
namespace mlad {

constexpr int kThreads = 192;
constexpr int kKeys = 64;          // keys per tile = one cache page = UMMA M of S^T
constexpr int kD = 576, kDV = 512;
constexpr int kBlocks = kD / 64;   // 9 dim blocks of 64
constexpr int kBlockBytes = kKeys * 128;
constexpr int kStageBytes = kBlocks * kBlockBytes;  // 72 KB
constexpr int kStages = 2;
constexpr int kMaxTickets = 1 << 16;
static __device__ int g_tickets[kMaxTickets];

struct Params {
  const void* q;
  void* out;
  float* ws_o;              // [splits, T, N, 512]
  float* ws_lse;            // [splits, T, N]
  const int* block_tables;
  const int* seq_lens;
  const int* qsl;
  int* status;
  unsigned long long* trace;  // optional phase timestamps [CTA][24] (null = off); slots 8-12 follow tile 4 through the pipeline, 13-19 the split merge
  int N, heads_per_cta, max_blocks, num_splits, early_meta;
  int cluster_merge;        // the num_splits CTAs of a (request, head group) form a cluster and merge in shared memory
  int64_t num_blocks, T;
  float scale_log2;
};

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float warp_max_redux(float v) {
  int i = __float_as_int(v);
  i = i >= 0 ? i : i ^ 0x7fffffff;
  i = __reduce_max_sync(0xffffffffu, i);
  i = i >= 0 ? i : i ^ 0x7fffffff;
  return __int_as_float(i);
}
__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

template <typename T> struct FmtOf;
template <> struct FmtOf<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct FmtOf<__half> { static constexpr uint32_t v = 0; };
template <typename T> __device__ __forceinline__ uint16_t to_bits16(float v);
template <> __device__ __forceinline__ uint16_t to_bits16<__nv_bfloat16>(float v) {
  return __bfloat16_as_ushort(__float2bfloat16(v));
}
template <> __device__ __forceinline__ uint16_t to_bits16<__half>(float v) { return __half_as_ushort(__float2half(v)); }

// R = UMMA N = rows of the Q^T operand (16 or 32): heads_per_cta * q_len <= R.
template <typename T, int R>
__global__ void __launch_bounds__(kThreads)
mla_decode_umma_kernel(const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ Params p) {
  constexpr int kQBytes = kBlocks * R * 128;   // Q^T operand: [9 dim blocks][R rows][128 B]
  constexpr int kPBytes = R * 128;             // one P buffer: [R rows][64 keys] 16-bit
  constexpr int kTmemCols = 256;               // 2 x R (S^T) + 4 x R (O^T) <= 192
  constexpr float kMaxSlack = 8.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + kStages * kStageBytes;
  uint8_t* sP = sQ + kQBytes;                  // [2][kPBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* kv_full = bars;                    // [2]
  uint64_t* kv_empty = bars + 2;               // [2]
  uint64_t* s_full = bars + 4;                 // [2]
  uint64_t* s_empty = bars + 6;                // [2]
  uint64_t* p_ready = bars + 8;                // [2]
  uint64_t* p_free = bars + 10;                // [2]
  uint64_t* o_done = bars + 12;                // [1]
  uint64_t* merge_bar = bars + 13;             // [1] bulk copies of the split merge
  uint64_t* o_final = bars + 14;               // [1] committed once, after the last P.V (epilogue wait)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* ok_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [4]
  int* s_last = reinterpret_cast<int*>(tmem_slot + 6);
  float* sMax = reinterpret_cast<float*>(tmem_slot + 8);   // [2][4 warps][R]
  float* sSum = sMax + 2 * 4 * R;                          // [4][R]
  float* sAlpha = sSum + 4 * R;                            // [R]
  float* sLse = sAlpha + R;                                // [16 splits][R]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Abort ab{p.status, abort_flag};
  const int cta_id = blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 0);  // start

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int b = 0; b < 2; ++b) {
      mbar_init(&kv_full[b], 1); mbar_init(&kv_empty[b], 1);
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4);
      mbar_init(&p_ready[b], 4); mbar_init(&p_free[b], 1);
    }
    mbar_init(o_done, 1);
    mbar_init(merge_bar, 1);
    mbar_init(o_final, 1);
    mbar_fence_init();
    prefetch_tmap(&tmKV);
    griddep_launch();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (!p.early_meta) griddep_wait();

  const int H = p.heads_per_cta;
  const int head0 = blockIdx.x * H;
  const int nh = min(H, p.N - head0);          // heads served by this CTA
  const int req = blockIdx.y / p.num_splits;
  const int split = blockIdx.y % p.num_splits;
  const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
  const int seq_len = p.seq_lens[req];
  const int rows_total = q_len * nh;           // row r = token r / nh, head r % nh
  const int ctx = seq_len - q_len;
  const int kv_end = seq_len;
  const bool served = q_len > 0 && rows_total <= R && nh > 0;
  const int n_tiles_all = served ? (kv_end + kKeys - 1) / kKeys : 0;
  const int per_split = (n_tiles_all + p.num_splits - 1) / p.num_splits;
  const int tile_lo = split * per_split;
  const int tile_hi = min(n_tiles_all, tile_lo + per_split);
  const int n_tiles = max(0, tile_hi - tile_lo);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_tiles > 0) {
      const int* bt = p.block_tables + (int64_t)req * p.max_blocks;
      bool ok = true, waited = p.early_meta == 0;
      int issued = 0;
      for (int i = 0; i < n_tiles; ++i) {
        const int stage = i & 1;
        const int page = tile_lo + i;
        const bool old_ctx = (page + 1) * kKeys <= ctx;
        if (!waited && (i >= kStages || !old_ctx)) { griddep_wait(); waited = true; }
        if (i >= kStages && !wait_or_abort(&kv_empty[stage], ((i >> 1) - 1) & 1, ab, 601)) { ok = false; break; }
        if (i == 4) trace_mark(p.trace, cta_id, 8);    // producer: stage of tile 4 is free
        mbar_expect_tx(&kv_full[stage], kStageBytes);
        int64_t blk = page < p.max_blocks ? bt[page] : 0;
        if (blk < 0 || blk >= p.num_blocks) blk = 0;
        uint8_t* dst = smem + stage * kStageBytes;
#pragma unroll
        for (int b = 0; b < kBlocks; ++b)
          tma_load_2d(dst + b * kBlockBytes, &tmKV, &kv_full[stage], b * 64, (int)(blk * kKeys));
        ++issued;
      }
      if (!ok) {
        for (int i = max(0, issued - kStages); i < issued; ++i)
          for (uint32_t q2 = 0; q2 < (1u << 16); ++q2)
            if (mbar_try_wait(&kv_full[i & 1], (i >> 1) & 1)) break;
      }
    }
    if (p.cluster_merge) {  // the two cluster barriers of the merge count every thread of every CTA
      __syncwarp();
      cluster_arrive(); cluster_wait();
      cluster_arrive(); cluster_wait();
    }
  } else {
    griddep_wait();
    // ---- Q^T operand (warps 1-5): [9 blocks][R rows][128 B]; 16-byte chunk c of row r sits at chunk c ^ (r & 7)
    // asynchronous 16-byte copies: every chunk of a thread is in flight at once (zero-filled past the last row)
    for (int c = threadIdx.x - 32; c < R * (kD / 8); c += kThreads - 32) {
      const int r = c / (kD / 8), ch = c % (kD / 8);
      const bool valid = r < rows_total && served;
      const int tok = valid ? r / nh : 0, hh = valid ? r % nh : 0;
      const T* src = reinterpret_cast<const T*>(p.q) + ((int64_t)(qs + tok) * p.N + head0 + hh) * kD + ch * 8;
      const int kb = ch / 8, cc = ch % 8;
      cp_async16(sQ + kb * (R * 128) + r * 128 + ((cc ^ (r & 7)) << 4), valid ? src : p.q, valid);
    }
    cp_async_commit();
    for (int c = threadIdx.x - 32; c < 2 * kPBytes / 16; c += kThreads - 32)
      reinterpret_cast<uint4*>(sP)[c] = make_uint4(0, 0, 0, 0);
    cp_async_wait<0>();
    fence_proxy_async_smem();
    named_bar_sync(2, kThreads - 32);
    if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 1);  // previous kernel done, Q staged
  }

  if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t fmt = FmtOf<T>::v;
      const uint32_t idesc_s = umma_idesc(kKeys, R, fmt, fmt, 0, 0);   // A = K page (K-major), B = Q^T (K-major)
      const uint32_t idesc_o = umma_idesc(128, R, fmt, fmt, 1, 0);     // A = V page (MN-major), B = P (K-major)
      const uint32_t tS = tmem_base, tO = tmem_base + 2 * R;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      // Event-driven: S^T of the next page and P.V of the current one do not depend on each other (the first waits
      // for its page to land, the second for the softmax warps), so whichever is ready is issued first.  Waiting
      // for them in a fixed order would hold P.V(i) - and with it the refill of its stage - behind the load of
      // page i + 1.
      auto issue_s = [&](int i) {
        const int stage = i & 1, buf = i & 1;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + stage * kStageBytes);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const int kb = k / 4, kk = k % 4;
          uint64_t da = umma_desc_k_sw128(k_addr + kb * kBlockBytes + kk * 32);
          uint64_t db = umma_desc_k_sw128(q_addr + kb * (R * 128) + kk * 32);
          umma_f16(tS + buf * R, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[buf]);
      };
      auto issue_pv = [&](int i) {
        const int pb = i & 1, stage = i & 1;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + stage * kStageBytes);
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k) {      // k outer: consecutive MMAs go to four different O^T tiles
#pragma unroll
          for (int j = 0; j < kDV / 128; ++j) {     // O^T tile j: dims [128 j, 128 j + 128) = blocks 2j, 2j + 1
            uint64_t da = umma_desc_mn_sw128(v_addr + (2 * j) * kBlockBytes + k * 2048, kBlockBytes, 1024);
            uint64_t db = umma_desc_k_sw128(p_addr + pb * kPBytes + k * 32);
            umma_f16(tO + j * R, da, db, idesc_o, (i > 0 || k > 0) ? 1u : 0u);
          }
        }
        // o_done first: whoever has seen p_free of this tile may rely on o_done having advanced as well
        umma_commit(o_done);
        umma_commit(&kv_empty[stage]);
        umma_commit(&p_free[pb]);
        if (i == n_tiles - 1) umma_commit(o_final);
      };
      int next_s = 0, next_pv = 0;
      uint32_t spins = 0;
      while (next_pv < n_tiles) {
        bool progressed = false;
        // S^T(next_s): its page has landed and its TMEM buffer has been read (at most one S^T ahead of P.V)
        if (next_s < n_tiles && next_s <= next_pv + 1 && mbar_try_wait(&kv_full[next_s & 1], (next_s >> 1) & 1) &&
            (next_s < 2 || mbar_try_wait(&s_empty[next_s & 1], ((next_s >> 1) - 1) & 1))) {
          if (next_s == 4) trace_mark(p.trace, cta_id, 9);    // issuer: tile 4 has landed
          issue_s(next_s);
          ++next_s;
          progressed = true;
        }
        if (next_pv < next_s && mbar_try_wait(&p_ready[next_pv & 1], (next_pv >> 1) & 1)) {
          if (next_pv == 4) trace_mark(p.trace, cta_id, 12);   // issuer: P of tile 4 is in shared memory
          issue_pv(next_pv);
          ++next_pv;
          progressed = true;
        }
        if (progressed) { spins = 0; continue; }
        if (++spins > (1u << 20)) { ab.raise(602); break; }
        if ((spins & 255) == 255 && ab.aborted()) break;
      }
    }
    if (p.cluster_merge) {
      __syncwarp();
      cluster_arrive(); cluster_wait();
      cluster_arrive(); cluster_wait();
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ softmax + epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int tid = (warp - 2) * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_off, tO = tmem_base + 2 * R + lane_off;
    const bool key_thread = lane < 16;               // an M = 64 accumulator uses lanes 0..15 of every quadrant
    const int key_in_tile = quarter * 16 + lane;     // valid when key_thread
    float m_used[R], l_part[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { m_used[r] = -INFINITY; l_part[r] = 0.f; }
    const int p_off = (key_in_tile & 7) * 2, p_ch = (key_in_tile & 63) >> 3;
    // One named barrier per tile in the common case.  Every thread polls the mbarriers itself (bounded); a thread whose
    // wait ran out keeps walking the loop with `fail` set, and the barrier below - which also tells whether any row's
    // running maximum has to move - makes all 128 threads leave together.
    bool ok = true, fail = false;
    for (int i = 0; i < n_tiles; ++i) {
      const int buf = i & 1;
      if (!fail && !wait_or_abort(&s_full[buf], (i >> 1) & 1, ab, 605)) fail = true;
      // P buffer i & 1 must have been consumed (P.V of tile i - 2).  Waiting here, before a possible rescale, also
      // keeps o_done at most one phase behind, so that the parity wait on it below cannot pass two phases early.
      if (i >= 2 && !fail && !wait_or_abort(&p_free[buf], ((i >> 1) - 1) & 1, ab, 606)) fail = true;
      tc_fence_after_sync();
      if (tid == 0 && i == 0) trace_mark(p.trace, cta_id, 2);  // first S^T ready
      if (tid == 0 && i == 4) trace_mark(p.trace, cta_id, 10);  // softmax: S^T of tile 4 ready
      float sc[R];
#pragma unroll
      for (int c = 0; c < R; c += 16) {
        uint32_t sr[16];
        tmem_ld_x16(tS + buf * R + c, sr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) sc[c + j] = __uint_as_float(sr[j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);
      const int key0 = (tile_lo + i) * kKeys;
      const int key = key0 + key_in_tile;
      const bool full = key0 + kKeys - 1 <= ctx && key0 + kKeys <= kv_end;
      bool need = fail;   // does any score exceed its row's reference maximum by more than the slack?
      if (full) {  // every key of the page is visible to every query token: no per-row positions needed
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float v = (key_thread && r < rows_total) ? sc[r] * p.scale_log2 : -INFINITY;
          sc[r] = v;
          need |= v > m_used[r] + kMaxSlack;
        }
      } else {
        int tok = 0, hh = 0;  // row r = token tok, head hh (walked without divisions)
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const bool in = key_thread && r < rows_total && key < kv_end && key <= ctx + tok;
          const float v = in ? sc[r] * p.scale_log2 : -INFINITY;
          sc[r] = v;
          need |= v > m_used[r] + kMaxSlack;
          if (++hh == nh) { hh = 0; ++tok; }
        }
      }
      if (bar_red_or(1, 128, need)) {
        // ---- rare after the first tiles: exchange the per-warp maxima, move the reference maxima, rescale O^T
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float wm = warp_max_redux(sc[r]);
          if (lane == (r & 31)) sMax[quarter * R + r] = wm;
        }
        const bool warp_failed = __any_sync(0xffffffffu, fail);
        if (lane == 0) ok_slot[quarter] = warp_failed ? 0 : 1;
        named_bar_sync(1, 128);
        if ((ok_slot[0] & ok_slot[1] & ok_slot[2] & ok_slot[3]) == 0) { ok = false; break; }
        float alpha[R];
        bool rescale = false;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float* mm = sMax + r;
          const float tm = fmaxf(fmaxf(mm[0], mm[R]), fmaxf(mm[2 * R], mm[3 * R]));
          alpha[r] = 1.f;
          if (tm > m_used[r] + kMaxSlack) {
            alpha[r] = exp2f(m_used[r] - tm);   // 0 when the row had no key yet
            m_used[r] = tm;
            l_part[r] *= alpha[r];
            rescale = true;
          }
        }
        if (rescale && i > 0) {   // same decision in every thread: all of them read the same maxima
          if (!wait_or_abort(o_done, (i - 1) & 1, ab, 608)) fail = true;
          tc_fence_after_sync();
#pragma unroll 1
          for (int j = 0; j < kDV / 128; ++j) {
#pragma unroll
            for (int c = 0; c < R; c += 16) {
              uint32_t orr[16];
              tmem_ld_x16(tO + j * R + c, orr);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) orr[e] = __float_as_uint(__uint_as_float(orr[e]) * alpha[c + e]);
              tmem_st_x16(tO + j * R + c, orr);
            }
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float ms = (m_used[r] == -INFINITY) ? 0.f : m_used[r];
        sc[r] = exp2f(sc[r] - ms);
        l_part[r] += sc[r];
      }
      if (key_thread && !fail) {
        uint8_t* base = sP + buf * kPBytes + p_off;
#pragma unroll
        for (int r = 0; r < R; ++r)
          *reinterpret_cast<uint16_t*>(base + r * 128 + ((p_ch ^ (r & 7)) << 4)) = to_bits16<T>(sc[r]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      const bool warp_failed = __any_sync(0xffffffffu, fail);
      __syncwarp();
      if (lane == 0 && !warp_failed) mbar_arrive(&p_ready[buf]);
      if (tid == 0 && i == 4) trace_mark(p.trace, cta_id, 11);  // softmax: P of tile 4 written
    }
    if (fail) ok = false;
    if (tid == 0) trace_mark(p.trace, cta_id, 3);  // last P written
    if (ok && n_tiles > 0) {
      // A parity wait on o_done would be wrong here: by now the barrier may be one phase short of the last P.V, at
      // it, or past it, and parity cannot tell the first from the last.  o_final completes exactly once.
      if (!wait_or_abort(o_final, 0, ab, 607)) ok = false;
      tc_fence_after_sync();
    }
    ok = bar_red_or(1, 128, !ok) == 0;   // one thread's time-out ends the tile for all
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float v = l_part[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == (r & 31)) sSum[quarter * R + r] = v;
    }
    named_bar_sync(1, 128);
    const int d = quarter * 32 + lane;               // output dim within an O^T tile (M = 128: lane = row)
    if (tid == 0) trace_mark(p.trace, cta_id, 4);  // last P.V done
    if (p.cluster_merge) {
      // ---- split merge inside the cluster: CTA c owns output dims [c * DS, (c + 1) * DS).  Every CTA stores its
      // un-normalised partial O (and per row its running maximum and sum) into the owners' shared memory, which
      // re-uses the cache-page stages once every CTA of the cluster has finished its last MMA (barrier A);
      // barrier B publishes the stores, then each owner combines S partials for its slice.  No global workspace,
      // no ticket, and the combine is spread over all CTAs instead of the last arriver.
      const int S = p.num_splits, DS = kDV / S;
      float* recv = reinterpret_cast<float*>(smem);                   // [S sources][R rows][DS dims]
      float* recv_ml = reinterpret_cast<float*>(smem + kStageBytes);  // [S sources][R rows][max, sum]
      cluster_arrive(); cluster_wait();  // A
      if (tid == 0) trace_mark(p.trace, cta_id, 5);
      if (served) {
        if (tid < R) {
          float m_mine = -INFINITY;  // m_used[tid] without a dynamically indexed register array
#pragma unroll
          for (int r = 0; r < R; ++r) m_mine = (tid == r) ? m_used[r] : m_mine;
          const float L = sSum[tid] + sSum[R + tid] + sSum[2 * R + tid] + sSum[3 * R + tid];
          const uint32_t local = smem_u32(recv_ml + (split * R + tid) * 2);
          for (int c = 0; c < S; ++c) {
            const uint32_t remote = mapa(local, (uint32_t)c);
            st_cluster_f32(remote, ok ? m_mine : -INFINITY);
            st_cluster_f32(remote + 4, ok ? L : 0.f);
          }
        }
#pragma unroll 1
        for (int j = 0; j < kDV / 128; ++j) {
          const int dim = j * 128 + d;
          const uint32_t remote = mapa(smem_u32(recv + (size_t)split * R * DS + dim % DS), (uint32_t)(dim / DS));
#pragma unroll
          for (int c = 0; c < R; c += 16) {
            uint32_t orr[16];
            if (ok && n_tiles > 0) {
              tmem_ld_x16(tO + j * R + c, orr);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) orr[e] = 0;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) st_cluster_f32(remote + (uint32_t)((c + e) * DS * 4), __uint_as_float(orr[e]));
          }
        }
      }
      cluster_arrive(); cluster_wait();  // B
      if (tid == 0) trace_mark(p.trace, cta_id, 6);
      // per row: the weight of every source (already divided by the common denominator) and the output row
      float* sW = sMax;                                   // [S][R] (the per-tile maxima are no longer needed)
      long long* sRow = reinterpret_cast<long long*>(smem + kStageBytes + 4096);  // [R]
      if (tid < R) {
        const int r = tid;
        float M = -INFINITY;
        for (int s2 = 0; s2 < S; ++s2) M = fmaxf(M, recv_ml[(s2 * R + r) * 2]);
        float den = 0.f;
        for (int s2 = 0; s2 < S; ++s2) {
          const float ms = recv_ml[(s2 * R + r) * 2];
          const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
          den = fmaf(recv_ml[(s2 * R + r) * 2 + 1], w, den);
          sW[s2 * R + r] = w;
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        for (int s2 = 0; s2 < S; ++s2) sW[s2 * R + r] *= inv;
        sRow[r] = (r < rows_total && served) ? (long long)(qs + r / nh) * p.N + head0 + r % nh : 0;
      }
      named_bar_sync(1, 128);
      if (served) {
        const int DS4 = DS / 4, sh = 31 - __clz(DS4);      // DS4 is a power of two (16, 32 or 64)
        for (int idx = tid; idx < rows_total * DS4; idx += 128) {
          const int r = idx >> sh, d4 = idx & (DS4 - 1);
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s2 = 0; s2 < S; ++s2) {
            const float w = sW[s2 * R + r];
            const float4 v = *reinterpret_cast<const float4*>(recv + ((size_t)s2 * R + r) * DS + d4 * 4);
            acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
            acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
          }
          alignas(8) T o4[4] = {from_float<T>(acc.x), from_float<T>(acc.y), from_float<T>(acc.z), from_float<T>(acc.w)};
          *reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.out) + sRow[r] * kDV + split * DS + d4 * 4) =
              *reinterpret_cast<const uint2*>(o4);
        }
      }
    } else if (served) {
      if (tid == 0) trace_mark(p.trace, cta_id, 5);  // row sums exchanged
      // per row, once: 1 / sum, the output row, the log-sum-exp (instead of divisions inside the store loops)
      float* sInv = sMax;                                                  // [R]
      long long* sRow = reinterpret_cast<long long*>(sMax + 2 * R);        // [R]
      if (tid < R) {
        const int r = tid;
        float m_mine = -INFINITY;
#pragma unroll
        for (int rr = 0; rr < R; ++rr) m_mine = (tid == rr) ? m_used[rr] : m_mine;
        const float L = sSum[r] + sSum[R + r] + sSum[2 * R + r] + sSum[3 * R + r];
        const int64_t orow = r < rows_total ? (int64_t)(qs + r / nh) * p.N + head0 + r % nh : 0;
        sInv[r] = (ok && L > 0.f) ? 1.f / L : 0.f;
        sRow[r] = orow;
        if (p.num_splits > 1 && r < rows_total)
          p.ws_lse[(int64_t)split * p.T * p.N + orow] = (ok && L > 0.f) ? m_mine + log2f(L) : -INFINITY;
      }
      named_bar_sync(1, 128);
      if (tid == 0) trace_mark(p.trace, cta_id, 16);
      T* outp = reinterpret_cast<T*>(p.out);
      float* wsp = p.ws_o + (int64_t)split * p.T * p.N * kDV;
#pragma unroll 1
      for (int j = 0; j < kDV / 128; ++j) {
#pragma unroll
        for (int c = 0; c < R; c += 16) {
          uint32_t orr[16];
          if (ok && n_tiles > 0) {
            tmem_ld_x16(tO + j * R + c, orr);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) orr[e] = 0;
          }
          // row scale and offset first, into registers: the compiler cannot move shared-memory loads across the
          // global stores below (both are generic pointers to it), and 16 load -> store chains in a row are slow
          float inv[16];
          int64_t off[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) { inv[e] = sInv[c + e]; off[e] = sRow[c + e] * kDV + j * 128 + d; }
          if (p.num_splits == 1) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (c + e < rows_total) outp[off[e]] = from_float<T>(__uint_as_float(orr[e]) * inv[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (c + e < rows_total) wsp[off[e]] = __uint_as_float(orr[e]) * inv[e];
          }
        }
      }
    }
    if (p.num_splits > 1 && !p.cluster_merge && served) {
      if (tid == 0) trace_mark(p.trace, cta_id, 17);
      __threadfence();
      if (tid == 0) trace_mark(p.trace, cta_id, 18);
      named_bar_sync(1, 128);
      const int ticket_idx = req * gridDim.x + blockIdx.x;
      if (tid == 0) *s_last = (atomicAdd(&g_tickets[ticket_idx], 1) == p.num_splits - 1);
      named_bar_sync(1, 128);
      if (tid == 0) trace_mark(p.trace, cta_id, 6);  // partial stored, ticket taken
      if (*s_last) {
        __threadfence();
        const int64_t sstride = p.T * p.N;
        const int S = p.num_splits;
        float* sW = sLse;                                   // [S][R]: log-sum-exps, then normalised weights
        const long long* sRow = reinterpret_cast<const long long*>(sMax + 2 * R);  // output rows (set in the epilogue)
        for (int idx = tid; idx < S * R; idx += 128) {
          const int s2 = idx / R, r = idx % R;
          sLse[idx] = r < rows_total ? __ldcg(p.ws_lse + s2 * sstride + sRow[r]) : -INFINITY;
        }
        named_bar_sync(1, 128);
        if (tid < R) {
          const int r = tid;
          float M = -INFINITY;
          for (int s2 = 0; s2 < S; ++s2) M = fmaxf(M, sLse[s2 * R + r]);
          float den = 0.f;
          for (int s2 = 0; s2 < S; ++s2) {
            const float l = sLse[s2 * R + r];
            const float w = (l == -INFINITY) ? 0.f : exp2f(l - M);
            den += w;
            sW[s2 * R + r] = w;
          }
          const float inv = den > 0.f ? 1.f / den : 0.f;
          for (int s2 = 0; s2 < S; ++s2) sW[s2 * R + r] *= inv;
        }
        named_bar_sync(1, 128);
        // The partials (S x rows x 2 KB, in L2) come in with bulk copies - a few per split, all in flight at once -
        // into the cache-page stages, G rows per pass; plain loads would keep far fewer bytes in flight from one SM.
        if (tid == 0) trace_mark(p.trace, cta_id, 13);  // merger: weights ready
        float* land = reinterpret_cast<float*>(smem);        // [S][G rows][512]
        const int G = max(1, min(rows_total, (kStages * kStageBytes / (kDV * 4)) / S));
        bool merged_ok = true;
        int pass = 0;
        for (int g0 = 0; g0 < rows_total; g0 += G, ++pass) {
          const int g1 = min(rows_total, g0 + G);
          if (warp == 2) {
            // the other CTAs' partials were acquired through the generic proxy (ticket + fence); order the bulk
            // copies, which read through the async proxy, behind that
            asm volatile("fence.proxy.async;" ::: "memory");
            if (lane == 0) mbar_expect_tx(merge_bar, (uint32_t)(S * (g1 - g0) * kDV * 4));
            __syncwarp();
            for (int s2 = lane; s2 < S; s2 += 32) {
              int r = g0;
              while (r < g1) {   // runs of consecutive output rows (one per query token) are contiguous in the workspace
                int e = r + 1;
                while (e < g1 && sRow[e] == sRow[e - 1] + 1) ++e;
                bulk_load_1d(land + ((size_t)s2 * G + (r - g0)) * kDV, p.ws_o + (s2 * sstride + sRow[r]) * kDV,
                             (uint32_t)((e - r) * kDV * 4), merge_bar);
                r = e;
              }
            }
          }
          if (!wait_or_abort(merge_bar, pass & 1, ab, 609)) merged_ok = false;
          if (bar_red_or(1, 128, !merged_ok)) break;
          if (tid == 0 && pass == 0) trace_mark(p.trace, cta_id, 14);  // merger: first pass landed
          for (int r = g0; r < g1; ++r) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int s2 = 0; s2 < S; ++s2) {
              const float w = sW[s2 * R + r];
              float4 v = *reinterpret_cast<const float4*>(land + ((size_t)s2 * G + (r - g0)) * kDV + tid * 4);
              if (!(w > 0.f)) v = make_float4(0.f, 0.f, 0.f, 0.f);  // an empty split's rows may hold anything
              acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
              acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
            }
            alignas(8) T o4[4] = {from_float<T>(acc.x), from_float<T>(acc.y), from_float<T>(acc.z), from_float<T>(acc.w)};
            *reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.out) + sRow[r] * kDV + tid * 4) =
                *reinterpret_cast<const uint2*>(o4);
          }
          if (tid == 0 && pass == 0) trace_mark(p.trace, cta_id, 19);
          named_bar_sync(1, 128);   // the next pass overwrites the landing buffer
        }
        if (tid == 0) g_tickets[ticket_idx] = 0;
        if (tid == 0) trace_mark(p.trace, cta_id, 15);  // merger: done
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 7);  // end
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int R>
static int launch_r(const Params& p, const CUtensorMap& tm, int B, int head_groups, cudaStream_t st) {
  auto kern = mla_decode_umma_kernel<T, R>;
  const size_t smem = 1024 + (size_t)kStages * kStageBytes + kBlocks * R * 128 + 2 * R * 128 + 4096 + 16 * R * 4;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (p.cluster_merge)
    return (int)launch_pdl_cluster(kern, dim3(head_groups, B * p.num_splits), dim3(kThreads), dim3(1, p.num_splits, 1),
                                   smem, st, tm, p);
  return (int)launch_pdl(kern, dim3(head_groups, B * p.num_splits), dim3(kThreads), smem, st, tm, p);
}

template <typename T, int R>
static int max_clusters_r(int S) {
  auto kern = mla_decode_umma_kernel<T, R>;
  const size_t smem = 1024 + (size_t)kStages * kStageBytes + kBlocks * R * 128 + 2 * R * 128 + 4096 + 16 * R * 4;
  if (ensure_dynamic_smem((const void*)kern, (int)smem) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, S * 64);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = S; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
  return n;
}

}  // namespace mlad
}  // namespace b200

// How many clusters of S CTAs of the MLA decode kernel (R = 16 or 32 operand rows) the current device holds at once;
// the host sizes the split count so that a launch is one wave.
extern "C" int b200_mla_decode_max_clusters(int R, int S, int dtype) {
  using namespace b200;
  if (S < 1 || S > 8) return 0;
  if (dtype == 2) return R == 16 ? mlad::max_clusters_r<__half, 16>(S) : mlad::max_clusters_r<__half, 32>(S);
  return R == 16 ? mlad::max_clusters_r<__nv_bfloat16, 16>(S) : mlad::max_clusters_r<__nv_bfloat16, 32>(S);
}

// Dense paged MLA decode on tcgen05 (see the header of this file).  `tmap`: the cache as a 2-D [blocks * 64, 576]
// 16-bit tensor with 64 x 64 boxes and 128-byte swizzle.  Serves block_size 64 and max_query_len <= 32; heads are
// processed in groups of R / max_query_len (R = 16 or 32).  Returns 3 for shapes it does not serve.
extern "C" int b200_mla_decode_umma(void* out, const void* q, const void* tmap, const int* block_tables,
                                    const int* seq_lens, const int* qsl, float* ws_o, float* ws_lse, int* status,
                                    int64_t T_, int B, int N, int block_size, int max_blocks, int64_t num_blocks,
                                    int max_query_len, int num_splits, float scale, int early_meta, int dtype,
                                    unsigned long long* trace, cudaStream_t st) {
  using namespace b200;
  if (B == 0 || T_ == 0) return 0;
  if (block_size != mlad::kKeys || max_query_len < 1 || max_query_len > 32 || num_splits < 1 || num_splits > 16) return 3;
  const int R = (N * max_query_len <= 16) ? 16 : 32;
  const int H = R / max_query_len;  // heads per CTA
  if (H < 1) return 3;
  const int groups = (N + H - 1) / H;
  // 2, 4 or 8 splits without a workspace: the splits of a (request, head group) are one cluster and merge on chip
  const bool cluster_merge = ws_o == nullptr && (num_splits == 2 || num_splits == 4 || num_splits == 8);
  if (num_splits > 1 && !cluster_merge && (ws_o == nullptr || (int64_t)B * groups > mlad::kMaxTickets)) return 2;
  mlad::Params p;
  p.cluster_merge = cluster_merge ? 1 : 0;
  p.q = q; p.out = out; p.ws_o = ws_o; p.ws_lse = ws_lse; p.block_tables = block_tables; p.seq_lens = seq_lens;
  p.qsl = qsl; p.status = status; p.trace = trace; p.N = N; p.heads_per_cta = H; p.max_blocks = max_blocks; p.num_splits = num_splits;
  p.early_meta = early_meta; p.num_blocks = num_blocks; p.T = T_;
  p.scale_log2 = scale * 1.4426950408889634f;
  const CUtensorMap& tm = *reinterpret_cast<const CUtensorMap*>(tmap);
  if (dtype == 1) return R == 16 ? mlad::launch_r<__nv_bfloat16, 16>(p, tm, B, groups, st)
                                 : mlad::launch_r<__nv_bfloat16, 32>(p, tm, B, groups, st);
  if (dtype == 2) return R == 16 ? mlad::launch_r<__half, 16>(p, tm, B, groups, st)
                                 : mlad::launch_r<__half, 32>(p, tm, B, groups, st);
  return 3;
}
