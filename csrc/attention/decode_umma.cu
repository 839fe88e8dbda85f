// Paged GQA decode attention on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA straight from the
// paged KV cache.
//
// Orientation ("swap A/B"): a decode step has only a handful of query rows per KV head (group size x query
// tokens <= 16) but thousands of keys, so the KEYS are the UMMA M side and the query rows the N side:
//     S^T[128 keys, 16 rows] = K_tile[128 keys, D] . Q^T            (A = K tile, K-major, as cached)
//     O^T[D dims,   16 rows] += V_tile^T[D dims, 128 keys] . P      (A = V tile, MN-major, as cached)
// Both accumulators live in TMEM with one lane per key (S^T) / per output dim (O^T) and 16 fp32 columns, so the
// tensor-core rows are always full, the online-softmax rescale of O is a 16-column TMEM round trip, and the final
// store is one coalesced 256-byte row of `out` per query row.
//
// One CTA serves one (request, kv head, kv split).  192 threads:
//   warp 0     TMA producer: per 128-key tile two cache pages x (K, V) x two 64-dim halves as 64x64 boxes
//              (128-byte swizzle) into a 3-stage ring; pages are looked up in the block table
//   warp 1     allocates TMEM, issues tcgen05.mma (one thread): S^T of tile i+1 is issued before P.V of tile i
//   warps 2-5  softmax: thread t owns key t of the tile (TMEM lane t): mask, tile max per row (redux + a
//              shared-memory exchange between the four warps), exp2, P^T to one of two shared-memory buffers
//              (16-bit, K-major, swizzled) for the second MMA; the same threads own output dim t in the epilogue
// Split-KV partials go through the fp32 workspace and are merged by the last CTA of a (request, head) to arrive.
// Every wait is bounded: on time-out the status word is set, the CTA drains its copies, frees TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/gemm_common.cuh"

namespace b200 {
namespace dattn {

constexpr int kThreads = 192;
constexpr int kTileKeys = 128;   // UMMA M
constexpr int kRows = 16;        // UMMA N: packed query rows (group x query tokens), zero padded
constexpr int kPage = 64;        // keys per TMA box = cache block granularity handled by one box
constexpr int kMaxTickets = 1 << 16;
static __device__ int g_tickets[kMaxTickets];

struct Params {
  const void* q;            // [T, Hq, D]
  void* out;                // [T, Hq, D]
  float* ws_o;              // [splits, T, Hq, D]
  float* ws_lse;            // [splits, T, Hq]
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;
  const int* qsl;
  const float* sinks;
  int* status;
  int Hq, Hkv, block_size, max_blocks, num_splits, window, num_stages;
  int early_meta;           // lengths / block table were written long before this launch: read them, and fetch
                            // old-context tiles, before the programmatic-dependency wait
  int64_t num_blocks, T;
  float scale_log2;
};

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// warp-wide float max through the integer reduction unit (order-preserving float <-> int map)
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

// D = head dim (128): K-blocks of 64 dims.  Shared memory per stage: K [D/64][128 keys][128 B] then V the same.
// NR = number of query rows that are computed (4, 8 or 16 >= group x query tokens); the UMMA N stays 16 with the
// rows beyond the real ones zero.
//
// Online softmax with a LAZY running maximum: the reference maximum m_used of a row only moves when a tile's
// maximum exceeds it by more than kMaxSlack (in log2 units), so p = exp2(s - m_used) stays below 2^kMaxSlack and the
// result O / l is unchanged; in the common case O^T needs no rescale and the softmax warps never wait for the
// previous P.V to finish - they run ahead into a second P buffer while the tensor core works.
template <typename T, int D, int NR>
__global__ void __launch_bounds__(kThreads)
decode_umma_kernel(const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ Params p) {
  constexpr int KB = D / 64;                       // 64-dim blocks
  constexpr int kHalfBytes = kTileKeys * 128;      // one 64-dim block of a 128-key tile
  constexpr int kOpBytes = KB * kHalfBytes;        // K (or V) of one tile
  constexpr int kStageBytes = 2 * kOpBytes;
  constexpr int kQBytes = KB * kRows * 128;        // Q^T operand: [D/64][16 rows][128 B]
  constexpr int kPBytes = (kTileKeys / 64) * kRows * 128;  // one P buffer: [2 key blocks][16 rows][128 B]
  constexpr int kTmemCols = 64;                    // S^T x 2 buffers (16 cols each) + O^T (16 cols)
  constexpr float kMaxSlack = 8.f;
  static_assert(D == 128, "one 128-lane O^T tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int num_stages = p.num_stages;
  uint8_t* sQ = smem + num_stages * kStageBytes;
  uint8_t* sP = sQ + kQBytes;                      // [2][kPBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* kv_full = bars;                        // [stages]
  uint64_t* kv_empty = bars + num_stages;          // [stages]
  uint64_t* s_full = bars + 2 * num_stages;        // [2]
  uint64_t* s_empty = s_full + 2;                  // [2]
  uint64_t* p_ready = s_empty + 2;                 // [2]
  uint64_t* p_free = p_ready + 2;                  // [2]
  uint64_t* o_done = p_free + 2;                   // [1] one phase per P.V (rescale waits, at most one phase behind)
  uint64_t* o_final = o_done + 1;                  // [1] committed once, after the last P.V (epilogue wait)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_final + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* ok_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [4]
  int* s_last = reinterpret_cast<int*>(tmem_slot + 6);
  float* sMax = reinterpret_cast<float*>(tmem_slot + 8);  // [2][4 warps][16 rows]
  float* sSum = sMax + 2 * 4 * kRows;                     // [4][16]
  float* sLse = sSum + 4 * kRows;                         // [16 splits][16 rows] (merge)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Abort ab{p.status, abort_flag};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < num_stages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4);
      mbar_init(&p_ready[b], 4); mbar_init(&p_free[b], 1);
    }
    mbar_init(o_done, 1);
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

  // With early_meta the request geometry comes from buffers the host filled before the step started (lengths, block
  // table): it does not depend on the kernels in front of this one, so it is read - and the tiles that lie wholly in
  // the old context are fetched - BEFORE the programmatic-dependency wait; only q and the cache rows of this step's
  // own tokens (positions >= ctx) are produced by the preceding kernels.  Without it (metadata written by a kernel
  // that may still be draining) everything waits first.
  if (!p.early_meta) griddep_wait();
  const int g = p.Hq / p.Hkv;
  const int kvh = blockIdx.x;
  const int req = blockIdx.y / p.num_splits;
  const int split = blockIdx.y % p.num_splits;
  const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
  const int seq_len = p.seq_lens[req];
  const int rows_total = q_len * g;
  const int ctx = seq_len - q_len;
  const int kv_end = seq_len;
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, ctx - p.window + 1) / kTileKeys * kTileKeys;
  const bool served = q_len > 0 && rows_total <= NR;
  const int n_tiles_all = served ? (kv_end - kv_begin + kTileKeys - 1) / kTileKeys : 0;
  const int per_split = (n_tiles_all + p.num_splits - 1) / p.num_splits;
  const int tile_lo = split * per_split;
  const int tile_hi = min(n_tiles_all, tile_lo + per_split);
  const int n_tiles = max(0, tile_hi - tile_lo);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (does not need Q)
    if (elect_one() && n_tiles > 0) {
      const int* bt = p.block_tables + (int64_t)req * p.max_blocks;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      bool waited = false;
      for (int i = 0; i < n_tiles; ++i) {
        const bool old_ctx = kv_begin + (tile_lo + i + 1) * kTileKeys <= ctx;  // no key of this step in the tile
        if (!waited && (i >= num_stages || !old_ctx)) {
          griddep_wait();
          waited = true;
        }
        if (i >= num_stages && !wait_or_abort(&kv_empty[stage], phase ^ 1, ab, 501)) { ok = false; break; }
        mbar_expect_tx(&kv_full[stage], kStageBytes);
        uint8_t* sK = smem + stage * kStageBytes;
        uint8_t* sV = sK + kOpBytes;
        const int key0 = kv_begin + (tile_lo + i) * kTileKeys;
#pragma unroll
        for (int pg = 0; pg < kTileKeys / kPage; ++pg) {
          const int key = key0 + pg * kPage;
          const int bi = key / p.block_size;
          int64_t blk = (key < kv_end && bi < p.max_blocks) ? bt[bi] : 0;
          if (blk < 0 || blk >= p.num_blocks) blk = 0;  // masked keys: any initialised page will do
          const int64_t rowK = ((blk * 2) * p.Hkv + kvh) * p.block_size + (key % p.block_size);
          const int64_t rowV = rowK + (int64_t)p.Hkv * p.block_size;
#pragma unroll
          for (int h = 0; h < KB; ++h) {
            tma_load_2d(sK + h * kHalfBytes + pg * (kPage * 128), &tmKV, &kv_full[stage], h * 64, (int)rowK);
            tma_load_2d(sV + h * kHalfBytes + pg * (kPage * 128), &tmKV, &kv_full[stage], h * 64, (int)rowV);
          }
        }
        ++issued;
        if (++stage == num_stages) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        int pending = issued < num_stages ? issued : num_stages;
        for (int i = 0; i < pending; ++i) {
          int s = (stage - 1 - i + 2 * num_stages) % num_stages;
          uint32_t ph = (s < stage) ? phase : (phase ^ 1);
          for (uint32_t q2 = 0; q2 < (1u << 16); ++q2)
            if (mbar_try_wait(&kv_full[s], ph)) break;
        }
      }
    }
  } else {
    griddep_wait();  // q (and everything these warps write) depends on the preceding kernels
    // ---- Q^T operand (warps 1-5): [D/64][16 rows][128 B], 16-byte chunk c of row r at chunk c ^ (r & 7)
    for (int c = threadIdx.x - 32; c < kRows * (D / 8); c += kThreads - 32) {
      const int r = c / (D / 8), ch = c % (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows_total && served) {
        const int tok = r / g, hh = r % g;
        v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) +
                                            ((int64_t)(qs + tok) * p.Hq + kvh * g + hh) * D + ch * 8);
      }
      const int kb = ch / 8, cc = ch % 8;
      *reinterpret_cast<uint4*>(sQ + kb * (kRows * 128) + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
    }
    // padded rows of both P buffers stay zero for the whole kernel
    for (int c = threadIdx.x - 32; c < 2 * kPBytes / 16; c += kThreads - 32)
      reinterpret_cast<uint4*>(sP)[c] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    named_bar_sync(2, kThreads - 32);
  }

  if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t fmt = FmtOf<T>::v;
      const uint32_t idesc_s = umma_idesc(kTileKeys, kRows, fmt, fmt, 0, 0);   // A = K (K-major), B = Q^T (K-major)
      const uint32_t idesc_o = umma_idesc(D, kRows, fmt, fmt, 1, 0);           // A = V (MN-major), B = P (K-major)
      const uint32_t tS = tmem_base, tO = tmem_base + 2 * kRows;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      // Event-driven: S^T of the next tile and P.V of the current one do not depend on each other (the first waits
      // for its tile to land, the second for the softmax warps), so whichever is ready is issued first; a fixed
      // order would hold P.V(i) - and the refill of its stage - behind the load of tile i + 1.
      auto issue_s = [&](int i) {
        const int stage = i % num_stages;
        const int buf = i & 1;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + stage * kStageBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const int kb = k / 4, kk = k % 4;
          uint64_t da = umma_desc_k_sw128(k_addr + kb * kHalfBytes + kk * 32);
          uint64_t db = umma_desc_k_sw128(q_addr + kb * (kRows * 128) + kk * 32);
          umma_f16(tS + buf * kRows, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[buf]);
      };
      auto issue_pv = [&](int i) {
        const int pb = i & 1;
        tc_fence_after_sync();
        const int stage = i % num_stages;
        const uint32_t v_addr = smem_u32(smem + stage * kStageBytes + kOpBytes);
#pragma unroll
        for (int k = 0; k < kTileKeys / 16; ++k) {
          // A: 16 keys (two 8-row groups of 1024 B) x D dims (64-dim blocks kHalfBytes apart)
          uint64_t da = umma_desc_mn_sw128(v_addr + k * 2048, kHalfBytes, 1024);
          uint64_t db = umma_desc_k_sw128(p_addr + pb * kPBytes + (k / 4) * (kRows * 128) + (k % 4) * 32);
          umma_f16(tO, da, db, idesc_o, (i > 0 || k > 0) ? 1u : 0u);
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
        // S^T(next_s): its tile has landed and its TMEM buffer has been read (at most one S^T ahead of P.V)
        if (next_s < n_tiles && next_s <= next_pv + 1 &&
            mbar_try_wait(&kv_full[next_s % num_stages], (next_s / num_stages) & 1) &&
            (next_s < 2 || mbar_try_wait(&s_empty[next_s & 1], ((next_s >> 1) - 1) & 1))) {
          issue_s(next_s);
          ++next_s;
          progressed = true;
        }
        if (next_pv < next_s && mbar_try_wait(&p_ready[next_pv & 1], (next_pv >> 1) & 1)) {
          issue_pv(next_pv);
          ++next_pv;
          progressed = true;
        }
        if (progressed) { spins = 0; continue; }
        if (++spins > (1u << 20)) { ab.raise(502); break; }
        if ((spins & 255) == 255 && ab.aborted()) break;
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ softmax + epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int tid = (warp - 2) * 32 + lane;          // 0..127 (named-barrier group)
    const int lane_id = quarter * 32 + lane;         // TMEM lane: key of the tile / output dim
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_off, tO = tmem_base + 2 * kRows + lane_off;
    float m_used[NR], l_part[NR];
    int pos[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      m_used[r] = -INFINITY;
      l_part[r] = 0.f;
      pos[r] = (r < rows_total) ? ctx + r / g : -1;  // position of the row's query token (-1: padded row)
    }
    const int pos_min = ctx, pos_max = ctx + max(q_len, 1) - 1;
    // byte offset of this key's column in a P buffer row
    const int p_off = (lane_id >> 6) * (kRows * 128) + (lane_id & 7) * 2;
    const int p_ch = (lane_id & 63) >> 3;
    // One named barrier per tile in the common case.  Every thread polls the mbarriers itself (bounded); a thread whose
    // wait ran out keeps walking the loop with `fail` set, and the barrier below - which also tells whether any row's
    // reference maximum has to move - makes all 128 threads leave together.
    bool ok = true, fail = false;
    for (int i = 0; i < n_tiles; ++i) {
      const int buf = i & 1;
      if (!fail && !wait_or_abort(&s_full[buf], (i >> 1) & 1, ab, 505)) fail = true;
      // P buffer i & 1 must have been consumed (P.V of tile i - 2).  Waiting here, before a possible rescale, also
      // keeps o_done at most one phase behind, so that the parity wait on it below cannot pass two phases early.
      if (i >= 2 && !fail && !wait_or_abort(&p_free[buf], ((i >> 1) - 1) & 1, ab, 506)) fail = true;
      tc_fence_after_sync();
      uint32_t sr[kRows];
      tmem_ld_x16(tS + buf * kRows, sr);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);
      // ---- mask (only on tiles that touch the causal / length / window edge)
      const int key0 = kv_begin + (tile_lo + i) * kTileKeys;
      const int key = key0 + lane_id;
      const bool full = key0 + kTileKeys - 1 <= pos_min && key0 + kTileKeys <= kv_end &&
                        (p.window <= 0 || key0 > pos_max - p.window);
      float sc[NR];
      bool need = fail;   // does any score exceed its row's reference maximum by more than the slack?
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        float v = __uint_as_float(sr[r]) * p.scale_log2;
        if (!full) {
          const bool in = key < kv_end && key <= pos[r] && (p.window <= 0 || key > pos[r] - p.window);
          v = in ? v : -INFINITY;
        } else if (NR > 4 && pos[r] < 0) {
          v = -INFINITY;
        }
        sc[r] = v;
        need |= v > m_used[r] + kMaxSlack;
      }
      if (bar_red_or(1, 128, need)) {
        // ---- rare after the first tiles: exchange the per-warp maxima, move the reference maxima, rescale O^T
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const float wm = warp_max_redux(sc[r]);
          if (lane == r) sMax[quarter * kRows + r] = wm;
        }
        const bool warp_failed = __any_sync(0xffffffffu, fail);
        if (lane == 0) ok_slot[quarter] = warp_failed ? 0 : 1;
        named_bar_sync(1, 128);
        if ((ok_slot[0] & ok_slot[1] & ok_slot[2] & ok_slot[3]) == 0) { ok = false; break; }
        float alpha[NR];
        bool rescale = false;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const float* mm = sMax + r;
          const float tm = fmaxf(fmaxf(mm[0], mm[kRows]), fmaxf(mm[2 * kRows], mm[3 * kRows]));
          alpha[r] = 1.f;
          if (tm > m_used[r] + kMaxSlack) {            // also the first finite maximum (m_used = -inf)
            alpha[r] = exp2f(m_used[r] - tm);          // exp2(-inf) = 0: nothing accumulated yet
            m_used[r] = tm;
            l_part[r] *= alpha[r];
            rescale = true;
          }
        }
        if (rescale && i > 0) {  // the same decision in every thread: all of them read the same maxima
          if (!wait_or_abort(o_done, (i - 1) & 1, ab, 508)) fail = true;
          tc_fence_after_sync();
          uint32_t orr[kRows];
          tmem_ld_x16(tO, orr);
          tmem_ld_wait();
#pragma unroll
          for (int r = 0; r < NR; ++r) orr[r] = __float_as_uint(__uint_as_float(orr[r]) * alpha[r]);
          tmem_st_x16(tO, orr);
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float ms = (m_used[r] == -INFINITY) ? 0.f : m_used[r];
        sc[r] = exp2f(sc[r] - ms);
        l_part[r] += sc[r];
      }
      // ---- P^T (B operand, K-major): element (row r, this thread's key)
      if (!fail) {
        uint8_t* base = sP + buf * kPBytes + p_off;
#pragma unroll
        for (int r = 0; r < NR; ++r)
          *reinterpret_cast<uint16_t*>(base + r * 128 + ((p_ch ^ (r & 7)) << 4)) = to_bits16<T>(sc[r]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      const bool warp_failed = __any_sync(0xffffffffu, fail);
      __syncwarp();
      if (lane == 0 && !warp_failed) mbar_arrive(&p_ready[buf]);
    }
    if (fail) ok = false;
    // ---- epilogue: O^T lane = output dim, 16 columns = query rows
    if (ok && n_tiles > 0) {
      // A parity wait on o_done would be wrong here: by now the barrier may be one phase short of the last P.V, at
      // it, or past it, and parity cannot tell the first from the last.  o_final completes exactly once.
      if (!wait_or_abort(o_final, 0, ab, 507)) ok = false;
      tc_fence_after_sync();
    }
    ok = bar_red_or(1, 128, !ok) == 0;   // one thread's time-out ends the tile for all
    // row sums: every thread holds the part of its own keys
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      float v = l_part[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == r) sSum[quarter * kRows + r] = v;
    }
    named_bar_sync(1, 128);
    // per row, once: 1 / denominator, the output row, the log-sum-exp (instead of divisions inside the store loop)
    float* sInv = sMax;                                                     // [16]
    long long* sRow = reinterpret_cast<long long*>(sMax + 2 * kRows);       // [16]
    if (served && tid < NR) {
      const int r = tid;
      float m_mine = -INFINITY;
#pragma unroll
      for (int rr = 0; rr < NR; ++rr) m_mine = (tid == rr) ? m_used[rr] : m_mine;
      const float L = sSum[r] + sSum[kRows + r] + sSum[2 * kRows + r] + sSum[3 * kRows + r];
      const float Ms = (m_mine == -INFINITY) ? 0.f : m_mine;
      const int hh = kvh * g + r % g;
      const int64_t orow = r < rows_total ? (int64_t)(qs + r / g) * p.Hq + hh : 0;
      float den = L;
      if (p.num_splits == 1 && p.sinks != nullptr && r < rows_total) den += exp2f(p.sinks[hh] * 1.4426950408889634f - Ms);
      sInv[r] = (ok && den > 0.f) ? 1.f / den : 0.f;
      sRow[r] = orow;
      if (p.num_splits > 1 && r < rows_total)
        p.ws_lse[(int64_t)split * p.T * p.Hq + orow] = (ok && L > 0.f) ? Ms + log2f(L) : -INFINITY;
    }
    named_bar_sync(1, 128);
    if (served) {
      uint32_t orr[kRows];
      if (ok && n_tiles > 0) {
        tmem_ld_x16(tO, orr);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int r = 0; r < kRows; ++r) orr[r] = 0;
      }
      const int d = lane_id;
      // scales and offsets into registers first: shared-memory loads do not move across the global stores below
      float inv[NR];
      int64_t off[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) { inv[r] = sInv[r]; off[r] = sRow[r] * D + d; }
      if (p.num_splits == 1) {
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (r < rows_total) reinterpret_cast<T*>(p.out)[off[r]] = from_float<T>(__uint_as_float(orr[r]) * inv[r]);
      } else {
        float* wsp = p.ws_o + (int64_t)split * p.T * p.Hq * D;
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (r < rows_total) wsp[off[r]] = __uint_as_float(orr[r]) * inv[r];
      }
    }
    if (p.num_splits > 1 && served) {
      // ---- split-KV merge by the last CTA of this (request, kv head) to arrive
      __threadfence();
      named_bar_sync(1, 128);
      const int ticket_idx = req * p.Hkv + kvh;
      if (tid == 0) *s_last = (atomicAdd(&g_tickets[ticket_idx], 1) == p.num_splits - 1);
      named_bar_sync(1, 128);
      if (*s_last) {
        __threadfence();
        const int d = lane_id;
        const int S = p.num_splits;
        const int64_t sstride = p.T * p.Hq;
        // all log-sum-exps of this (request, head) in one round of loads: thread t -> (split t / 16, row t % 16)
        for (int idx = tid; idx < S * kRows; idx += 128) {
          const int s2 = idx / kRows, r = idx % kRows;
          sLse[idx] = (r < rows_total) ? __ldcg(p.ws_lse + s2 * sstride + sRow[r]) : -INFINITY;
        }
        named_bar_sync(1, 128);
        // weights, already divided by the common denominator (plus the sink's share), once per row
        float* sW = sLse;
        if (tid < NR && tid < rows_total) {
          const int r = tid;
          float M = -INFINITY;
          for (int s2 = 0; s2 < S; ++s2) M = fmaxf(M, sLse[s2 * kRows + r]);
          const float Ms = (M == -INFINITY) ? 0.f : M;
          float den = 0.f;
          for (int s2 = 0; s2 < S; ++s2) {
            const float l = sLse[s2 * kRows + r];
            const float w = (l == -INFINITY) ? 0.f : exp2f(l - Ms);
            den += w;
            sW[s2 * kRows + r] = w;
          }
          if (p.sinks != nullptr) den += exp2f(p.sinks[kvh * g + r % g] * 1.4426950408889634f - Ms);
          const float inv = den > 0.f ? 1.f / den : 0.f;
          for (int s2 = 0; s2 < S; ++s2) sW[s2 * kRows + r] *= inv;
        }
        named_bar_sync(1, 128);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          if (r >= rows_total) break;
          const float* src = p.ws_o + sRow[r] * D + d;
          float acc = 0.f;
          int s2 = 0;
          for (; s2 + 4 <= S; s2 += 4) {  // four independent loads in flight
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcg(src + (s2 + u) * sstride * D);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float w = sW[(s2 + u) * kRows + r];
              acc += w > 0.f ? v[u] * w : 0.f;   // an empty split's row may hold anything
            }
          }
          for (; s2 < S; ++s2) {
            const float w = sW[s2 * kRows + r];
            const float v = __ldcg(src + s2 * sstride * D);
            acc += w > 0.f ? v * w : 0.f;
          }
          reinterpret_cast<T*>(p.out)[sRow[r] * D + d] = from_float<T>(acc);
        }
        if (tid == 0) g_tickets[ticket_idx] = 0;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int NR>
static int launch_nr(const Params& p0, const CUtensorMap& tm, int B, cudaStream_t st) {
  constexpr int D = 128;
  auto kern = decode_umma_kernel<T, D, NR>;
  Params p = p0;
  constexpr int kStageBytes = 2 * (D / 64) * kTileKeys * 128;
  p.num_stages = 3;
  const size_t smem = 1024 + (size_t)p.num_stages * kStageBytes + (D / 64) * kRows * 128 + 2 * 2 * kRows * 128 + 4096;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)launch_pdl(kern, dim3(p.Hkv, B * p.num_splits), dim3(kThreads), smem, st, tm, p);
}

template <typename T>
static int launch(const Params& p, const CUtensorMap& tm, int B, int max_rows, cudaStream_t st) {
  if (max_rows <= 4) return launch_nr<T, 4>(p, tm, B, st);
  if (max_rows <= 8) return launch_nr<T, 8>(p, tm, B, st);
  return launch_nr<T, 16>(p, tm, B, st);
}

}  // namespace dattn
}  // namespace b200

// Decode-shaped paged attention (at most 16 packed query rows per KV head, head dim 128, cache blocks that are a
// multiple of 64 tokens) on tcgen05.  `tmap` describes the cache as a 2-D [blocks * 2 * Hkv * block_size, 128]
// 16-bit tensor with 64 x 64 boxes and 128-byte swizzle.  Returns 3 when the shape is not served.
extern "C" int b200_decode_attention_umma(void* out, const void* q, const void* tmap, const int* block_tables,
                                          const int* seq_lens, const int* qsl, const float* sinks, float* ws_o,
                                          float* ws_lse, int* status, int64_t T_, int B, int Hq, int Hkv, int D,
                                          int block_size, int max_blocks, int64_t num_blocks, int max_query_len,
                                          int num_splits, int window, float scale, int early_meta, int dtype,
                                          cudaStream_t st) {
  using namespace b200;
  if (B == 0 || T_ == 0) return 0;
  if (D != 128 || Hq % Hkv || max_query_len * (Hq / Hkv) > dattn::kRows || block_size % dattn::kPage) return 3;
  if (num_splits < 1 || num_splits > 16 ||
      (num_splits > 1 && (ws_o == nullptr || (int64_t)B * Hkv > dattn::kMaxTickets)))
    return 2;
  dattn::Params p;
  p.q = q; p.out = out; p.ws_o = ws_o; p.ws_lse = ws_lse; p.block_tables = block_tables; p.seq_lens = seq_lens;
  p.qsl = qsl; p.sinks = sinks; p.status = status; p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size;
  p.max_blocks = max_blocks; p.num_splits = num_splits; p.window = window; p.num_blocks = num_blocks; p.T = T_;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_stages = 3;
  p.early_meta = early_meta;
  const CUtensorMap& tm = *reinterpret_cast<const CUtensorMap*>(tmap);
  const int max_rows = max_query_len * (Hq / Hkv);
  if (dtype == 1) return dattn::launch<__nv_bfloat16>(p, tm, B, max_rows, st);
  if (dtype == 2) return dattn::launch<__half>(p, tm, B, max_rows, st);
  return 3;
}
