// Lightning-indexer logits for prefill-sized batches on tcgen05 + TMEM, fed by TMA.
//
//   logits[t, key] = k_scale[key] * sum_h  w[t, h] * relu( q8[t, h, :] . k8[key, :] )        key < n_keys(t)
//
// (the reference's `_C::I8_mqa_logits`, ops/deep_gemm.py:5-121; q8 / k8 are e4m3, w carries head weight x q scale).
// The contraction is a GEMM with the KEYS on the UMMA M side and (token, head) pairs on the N side:
//     D[128 keys, 4 tokens x 64 heads] = K_tile[128 keys, 128 dims] . Q_group^T            (kind::f8f6f4, 4 k-steps)
// so that one thread of the epilogue owns one key row: it applies ReLU, multiplies by the head weights, sums the 64
// heads of each of the 4 tokens out of its TMEM lane, multiplies by the key's scale and stores 4 logits.
// One CTA = (request, block of 16 consecutive query tokens of that request).  The block's Q operand (4 groups x
// 32 KB) stays resident in shared memory; key tiles (two 64-row cache pages, 16 KB) stream through a 3-stage ring,
// so the key cache of a request is read once per 16 query tokens and Q once.  Key pages come straight out of the
// page-major indexer cache: a block is 64 rows of 128 bytes followed by 256 bytes of scales = 66 rows of a
// [blocks * 66, 128]-byte matrix, which one 2-D tensor map with 128-byte swizzle covers.
// Two D buffers of 256 TMEM columns let the tensor core run a group ahead of the epilogue warps.
// 192 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue.  TMA loads carry no cluster multicast.
// Every wait is bounded; on time-out the status word is set and the CTA unwinds.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>

#include <algorithm>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/gemm_common.cuh"

namespace b200 {
namespace idxu {

// 32 consecutive TMEM columns of this thread's lane into r[0..31] (pointer form: the caller indexes one big array)
__device__ __forceinline__ void tmem_ld_x32_p(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

constexpr int kThreads = 192;
constexpr int kH = 64, kD = 128;             // heads, dims (bytes per e4m3 row)
constexpr int kTok = 16, kGroupTok = 4;      // query tokens per CTA / per MMA group
constexpr int kGroups = kTok / kGroupTok;
constexpr int kGroupN = kGroupTok * kH;      // 256 = UMMA N
constexpr int kKeyTile = 128, kPage = 64;
constexpr int kGroupBytes = kGroupN * kD;    // 32 KB
constexpr int kStageBytes = kKeyTile * kD;   // 16 KB
constexpr int kStages = 3;
constexpr int kBlockRows = 66;               // a cache block = 66 rows of 128 bytes (64 key rows + 2 rows of scales)
constexpr int kTmemCols = 512;

struct Params {
  float* logits;             // [rows, ld]
  const float* w;            // [rows, 64]
  const uint8_t* cache;      // [blocks][64 * 132] bytes
  const int* block_tables;   // [B, max_blocks]
  const int* seq_lens;       // [B]
  const int* qsl;            // [B + 1]
  int* status;
  int64_t ld, t_lo, t_hi;    // rows are tokens t_lo .. t_hi of the batch
  int64_t num_blocks;
  int max_blocks;
};

__global__ void __launch_bounds__(kThreads)
indexer_logits_umma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // [4 groups][256 rows][128 B]
  uint8_t* sK = sQ + kGroups * kGroupBytes;             // [3 stages][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sK + kStages * kStageBytes);
  uint64_t* q_full = bars;                              // [1]
  uint64_t* k_full = bars + 1;                          // [3]
  uint64_t* k_empty = bars + 4;                         // [3]
  uint64_t* d_full = bars + 7;                          // [2]
  uint64_t* d_empty = bars + 9;                         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* sW = reinterpret_cast<float*>(bars + 16);      // [16 tokens][64 heads], 16-byte aligned
  int* sNk = reinterpret_cast<int*>(sW + kTok * kH);    // [16] keys visible to each token (0: no such token)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Abort ab{p.status, abort_flag};
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&d_full[b], 1); mbar_init(&d_empty[b], 4); }
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
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
  griddep_wait();   // q, w and the key cache come from the preceding kernels

  // ---- this CTA's tokens: block blockIdx.x of request blockIdx.y, clipped to the rows [t_lo, t_hi)
  const int req = blockIdx.y;
  const int qs = p.qsl[req], qe = p.qsl[req + 1];
  const int seq_len = p.seq_lens[req];
  const int64_t first = max((int64_t)qs, p.t_lo), last = min((int64_t)qe, p.t_hi);
  const int64_t tb = first + (int64_t)blockIdx.x * kTok;           // first token of the block (batch index)
  const int n_tok = (int)max((int64_t)0, min((int64_t)kTok, last - tb));
  // keys visible to token t: seq_len - q_len + (t - qs) + 1; the block's last token sees the most
  const int nk_first = seq_len - (qe - qs) + (int)(tb - qs) + 1;
  const int nk_max = n_tok > 0 ? nk_first + n_tok - 1 : 0;
  const int n_tiles = (nk_max + kKeyTile - 1) / kKeyTile;
  const int n_groups = (n_tok + kGroupTok - 1) / kGroupTok;
  const int64_t row0 = tb - p.t_lo;                                // first logits / q / w row of the block

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_tiles > 0) {
      mbar_expect_tx(q_full, (uint32_t)(n_groups * kGroupBytes));
      for (int g = 0; g < n_groups; ++g)
        tma_load_2d(sQ + g * kGroupBytes, &tmQ, q_full, 0, (int)((row0 + g * kGroupTok) * kH));
      const int* bt = p.block_tables + (int64_t)req * p.max_blocks;
      int issued = 0;
      bool ok = true;
      for (int kt = 0; kt < n_tiles; ++kt) {
        const int stage = kt % kStages;
        if (kt >= kStages && !wait_or_abort(&k_empty[stage], ((kt / kStages) - 1) & 1, ab, 701)) { ok = false; break; }
        mbar_expect_tx(&k_full[stage], kStageBytes);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int page = kt * 2 + h;
          int64_t blk = page < p.max_blocks ? bt[page] : 0;   // beyond the request: any valid page (masked later)
          if (blk < 0 || blk >= p.num_blocks) blk = 0;
          tma_load_2d(sK + stage * kStageBytes + h * (kPage * kD), &tmK, &k_full[stage], 0, (int)(blk * kBlockRows));
        }
        ++issued;
      }
      if (!ok) {  // drain what is in flight before leaving
        for (int kt = max(0, issued - kStages); kt < issued; ++kt)
          for (uint32_t q2 = 0; q2 < (1u << 16); ++q2)
            if (mbar_try_wait(&k_full[kt % kStages], (kt / kStages) & 1)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t idesc = umma_idesc(kKeyTile, kGroupN, 0, 0);   // e4m3 x e4m3, both K-major
      bool ok = wait_or_abort(q_full, 0, ab, 702);
      int it = 0;
      for (int kt = 0; ok && kt < n_tiles; ++kt) {
        const int stage = kt % kStages;
        if (!wait_or_abort(&k_full[stage], (kt / kStages) & 1, ab, 703)) break;
        const uint32_t k_addr = smem_u32(sK + stage * kStageBytes);
        for (int g = 0; g < n_groups; ++g, ++it) {
          const int buf = it & 1;
          if (it >= 2 && !wait_or_abort(&d_empty[buf], ((it >> 1) - 1) & 1, ab, 704)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t q_addr = smem_u32(sQ + g * kGroupBytes);
#pragma unroll
          for (int kk = 0; kk < kD / 32; ++kk)
            umma_f8(tmem_base + buf * kGroupN, umma_desc_k_sw128(k_addr + kk * 32), umma_desc_k_sw128(q_addr + kk * 32),
                    idesc, kk > 0 ? 1u : 0u);
          umma_commit(&d_full[buf]);
        }
        if (ok) umma_commit(&k_empty[stage]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5): thread = key row
    const int quarter = warp & 3;
    const int tid = (warp - 2) * 32 + lane;
    const int r = quarter * 32 + lane;                 // TMEM lane = key within the tile
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    for (int i = tid; i < kTok * kH; i += 128) {
      const int tok = i / kH;
      sW[i] = tok < n_tok ? p.w[(row0 + tok) * kH + (i % kH)] : 0.f;
    }
    if (tid < kTok) sNk[tid] = tid < n_tok ? nk_first + tid : 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int* bt = p.block_tables + (int64_t)req * p.max_blocks;
    auto key_scale = [&](int kt) -> float {  // scale of this thread's key in tile kt (pages 2 kt, 2 kt + 1)
      const int page = kt * 2 + (r >> 6);
      int64_t blk = page < p.max_blocks ? bt[page] : 0;
      if (blk < 0 || blk >= p.num_blocks) blk = 0;
      return reinterpret_cast<const float*>(p.cache + blk * (kBlockRows * kD) + kPage * kD)[r & 63];
    };
    float sc_next = n_tiles > 0 ? key_scale(0) : 0.f;
    bool fail = false;
    int it = 0;
    for (int kt = 0; kt < n_tiles && !fail; ++kt) {
      const float sc = sc_next;
      if (kt + 1 < n_tiles) sc_next = key_scale(kt + 1);   // one tile ahead: no dependent load in front of the math
      const int key = kt * kKeyTile + r;
      for (int g = 0; g < n_groups; ++g, ++it) {
        const int buf = it & 1;
        if (!wait_or_abort(&d_full[buf], (it >> 1) & 1, ab, 705)) { fail = true; break; }
        tc_fence_after_sync();
        // A tcgen05.ld + wait pair costs a few hundred nanoseconds whatever its width: 128 columns (two tokens) per
        // round trip; four partial sums per token so that the FMAs do not wait on one another.
        float out4[kGroupTok];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[128];
#pragma unroll
          for (int c = 0; c < 128; c += 32) tmem_ld_x32_p(taddr + buf * kGroupN + half * 128 + c, v + c);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const int j = half * 2 + jj;
            const float* wj = sW + (g * kGroupTok + j) * kH;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < kH; e += 4) {
              const float4 w4 = *reinterpret_cast<const float4*>(wj + e);
              acc[0] = fmaf(fmaxf(__uint_as_float(v[jj * kH + e]), 0.f), w4.x, acc[0]);
              acc[1] = fmaf(fmaxf(__uint_as_float(v[jj * kH + e + 1]), 0.f), w4.y, acc[1]);
              acc[2] = fmaf(fmaxf(__uint_as_float(v[jj * kH + e + 2]), 0.f), w4.z, acc[2]);
              acc[3] = fmaf(fmaxf(__uint_as_float(v[jj * kH + e + 3]), 0.f), w4.w, acc[3]);
            }
            out4[j] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * sc;
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&d_empty[buf]);
#pragma unroll
        for (int j = 0; j < kGroupTok; ++j) {
          const int tok = g * kGroupTok + j;
          const int nk = sNk[tok];
          if (nk > 0 && key < p.ld) p.logits[(row0 + tok) * p.ld + key] = key < nk ? out4[j] : -INFINITY;
        }
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

}  // namespace idxu
}  // namespace b200

// Indexer logits of rows [t_lo, t_hi) of the batch on tcgen05 (block_size 64 only).  `tmQ`: q8 viewed as
// [rows * 64, 128] bytes with 256-row boxes; `tmK`: the cache viewed as [blocks * 66, 128] bytes with 64-row boxes;
// both with 128-byte swizzle.  Only keys [0, n_keys(t)) of a row are written, rounded up to the key tile (-inf there).
extern "C" int b200_indexer_logits_umma(float* logits, const void* tmQ, const float* w, const void* cache, const void* tmK,
                                        const int* block_tables, const int* seq_lens, const int* qsl, int* status,
                                        int B, int max_query_len, int max_blocks, int64_t num_blocks, int64_t ld,
                                        int64_t t_lo, int64_t t_hi, cudaStream_t st) {
  using namespace b200;
  if (B == 0 || t_hi <= t_lo || max_query_len <= 0) return 0;
  idxu::Params p;
  p.logits = logits; p.w = w; p.cache = (const uint8_t*)cache; p.block_tables = block_tables; p.seq_lens = seq_lens;
  p.qsl = qsl; p.status = status; p.ld = ld; p.t_lo = t_lo; p.t_hi = t_hi; p.num_blocks = num_blocks;
  p.max_blocks = max_blocks;
  const size_t smem = 1024 + idxu::kGroups * idxu::kGroupBytes + idxu::kStages * idxu::kStageBytes + 256 +
                      idxu::kTok * idxu::kH * 4 + 128;
  auto kern = idxu::indexer_logits_umma_kernel;
  cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int64_t span = std::min<int64_t>(max_query_len, t_hi - t_lo);
  dim3 grid((unsigned)((span + idxu::kTok - 1) / idxu::kTok), (unsigned)B);
  return (int)launch_pdl(kern, grid, dim3(idxu::kThreads), smem, st, *reinterpret_cast<const CUtensorMap*>(tmQ),
                         *reinterpret_cast<const CUtensorMap*>(tmK), p);
}
