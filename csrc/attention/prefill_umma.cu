// Paged GQA prefill / chunked-prefill attention on tcgen05 + TMEM, fed by TMA straight from the paged KV cache
// (head_dim 128, 16-bit).  The reference's `prefill_attention` call (v1/attention/backends/kunlun_attn.py:805-947).
//
// One CTA = (tile of 128 query rows of one request, one query head).  Per 128-key tile:
//     S[128 q rows, 128 keys]  = Q_tile[128, D] . K_tile^T             (A = Q, B = K tile, both K-major)
//     O[128 q rows, D]        += P[128, 128 keys] . V_tile[128 keys, D] (A = P from shared memory, B = V tile MN-major)
// S lives in TMEM with one lane per query row, so a softmax thread owns a whole row: row maximum, exp2 and row sum
// need no cross-thread exchange, and the online-softmax rescale of O is a round trip through the thread's own TMEM
// lane.  The running maximum is lazy (it moves only when a tile exceeds it by more than 8 in log2 units), so in the
// common case O is not rescaled and the softmax warps never wait for the previous P.V.
// 192 threads: warp 0 TMA producer (Q once; per key tile two cache pages x (K, V) x two 64-dim halves as 64 x 64
// boxes with 128-byte swizzle, 2-stage ring), warp 1 MMA issuer (event-driven: S of the next tile and P.V of the
// current one are issued as they become ready), warps 2-5 softmax + epilogue.  Two S buffers (2 x 128 TMEM columns)
// + O (128 columns).  Causal masking by position (chunked prefill: row r of the request sits at ctx + r), optional
// sliding window and attention sinks, optional log-sum-exp output.
// The MLA instantiation (`kMla`) is the compute-friendly prefill form of multi-head latent attention
// (v1/attention/backends/mla/common.py:1782-1843): 192-dim q / k (128 "nope" dims per head + 64 rotary dims shared
// by all heads), 128-dim v, keys and values read as contiguous rows of the up-projected `kv_b_proj` output
// ([rows, heads * 256], k_nope | v per head) plus the rotary key rows ([rows, 64]); each request's keys start at
// `kv_starts[req]`.  Causal (new tokens) or not (a chunk of cached context); the log-sum-exp output lets the caller
// merge chunks.  Its K ring has two 48 KB stages and V a single 32 KB one (208 KB of shared memory in all).
// TMA loads carry no cluster multicast.  Every wait is bounded; on time-out the status word is set and the CTA unwinds.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/gemm_common.cuh"

namespace b200 {
namespace pattn {

constexpr int kThreads = 192;
constexpr int kQTile = 128, kKTile = 128, kPage = 64, kD = 128;
constexpr int kHalfBytes = 128 * 128;          // one 64-dim block of a 128-row operand tile
constexpr int kOpBytes = 2 * kHalfBytes;       // Q, K, V or P tile: 32 KB
constexpr int kStages = 2;                     // K ring
template <bool kMla> struct Cfg {
  static constexpr int kQBlocks = kMla ? 3 : 2;                 // 64-dim blocks of q / k
  static constexpr int kKBytes = kQBlocks * kHalfBytes;         // Q tile or one K stage
  static constexpr int kVStages = kMla ? 1 : 2;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kKBytes + (size_t)kVStages * kOpBytes + kKBytes + kOpBytes + 256;
};
constexpr int kTmemCols = 512;                 // 2 x 128 (S) + 128 (O)
constexpr float kMaxSlack = 8.f;

struct Params {
  void* out;                // [T, Hq, 128]
  float* lse;               // [T, Hq] natural-log sum-exp (optional)
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;
  const int* qsl;
  const int* kv_starts;     // MLA form: first key row of each request in the contiguous K / V tensors
  const float* sinks;       // [Hq] or null
  int* status;
  unsigned long long* trace;   // optional phase timestamps [CTA][24] (null = off)
  int Hq, Hkv, block_size, max_blocks, window, causal;
  int64_t num_blocks;
  float scale_log2;
};

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

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
__device__ __forceinline__ void tmem_st_x32_p(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 2^x on the special-function unit (one instruction; -inf -> 0; -inf + -inf stays -inf, NaN cannot arise from the
// callers' finite-or-minus-infinity inputs with a finite or minus-infinity offset)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> struct FmtOf;
template <> struct FmtOf<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct FmtOf<__half> { static constexpr uint32_t v = 0; };
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16(a)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(b)) << 16);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  return (uint32_t)__half_as_ushort(__float2half(a)) | ((uint32_t)__half_as_ushort(__float2half(b)) << 16);
}

template <typename T, bool kMla>
__global__ void __launch_bounds__(kThreads)
prefill_umma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                    const __grid_constant__ CUtensorMap tmKpe, const __grid_constant__ Params p) {
  constexpr int kQBlocks = Cfg<kMla>::kQBlocks, kKBytes = Cfg<kMla>::kKBytes, kVStages = Cfg<kMla>::kVStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sVr = smem + kStages * kKBytes;          // V ring: [kVStages][2 dim blocks][128 keys][128 B]
  uint8_t* sQ = sVr + kVStages * kOpBytes;          // [kQBlocks dim blocks][128 rows][128 B]
  uint8_t* sP = sQ + kKBytes;                       // [2 key blocks][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kOpBytes);
  uint64_t* q_full = bars;             // [1]
  uint64_t* k_full = bars + 1;         // [2]
  uint64_t* k_empty = bars + 3;        // [2] S of the tile has been computed
  uint64_t* s_full = bars + 5;         // [2]
  uint64_t* s_empty = bars + 7;        // [2]
  uint64_t* p_ready = bars + 9;        // [1] 4 arrivals (one per softmax warp)
  uint64_t* p_free = bars + 10;        // [1]
  uint64_t* o_done = bars + 11;        // [1] one phase per P.V
  uint64_t* o_final = bars + 12;       // [1] once, after the last P.V
  uint64_t* v_full = bars + 13;        // [2] (kVStages used)
  uint64_t* v_empty = bars + 15;       // [2] P.V of the tile has been computed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Abort ab{p.status, abort_flag};
  const int cta_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 0);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 1); mbar_init(&k_empty[b], 1);
      mbar_init(&v_full[b], 1); mbar_init(&v_empty[b], 1);
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4);
    }
    mbar_init(p_ready, 4); mbar_init(p_free, 1); mbar_init(o_done, 1); mbar_init(o_final, 1);
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmKV);
    if (kMla) prefetch_tmap(&tmKpe);
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
  griddep_wait();   // q and this step's cache rows come from the preceding kernels

  const int head = blockIdx.y, req = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  const int qs = p.qsl[req], q_len = p.qsl[req + 1] - qs;
  const int seq_len = p.seq_lens[req];
  // not causal: every row sees all of the request's keys - as if it sat far behind them
  const int ctx = (kMla && !p.causal) ? (1 << 29) : seq_len - q_len;
  const int row0 = blockIdx.x * kQTile;                      // first query row of this tile within the request
  const int n_rows = max(0, min(kQTile, q_len - row0));
  // keys visible to the tile: up to the position of its last row; with a window, from the first row's window start
  const int pos_first = ctx + row0, pos_last = ctx + row0 + n_rows - 1;
  const int kv_end = n_rows > 0 ? min(seq_len, pos_last + 1) : 0;
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, pos_first - p.window + 1) / kKTile * kKTile;
  const int n_tiles = n_rows > 0 ? (kv_end - kv_begin + kKTile - 1) / kKTile : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_tiles > 0) {
      mbar_expect_tx(q_full, kKBytes);
#pragma unroll
      for (int h = 0; h < kQBlocks; ++h)
        tma_load_2d(sQ + h * kHalfBytes, &tmQ, q_full, head * (kQBlocks * 64) + h * 64, qs + row0);
      const int* bt = kMla ? nullptr : p.block_tables + (int64_t)req * p.max_blocks;
      const int kv_row0 = kMla ? p.kv_starts[req] : 0;
      // cache row of a key's page (paged form): masked keys read any initialised page
      auto page_row = [&](int key) -> int64_t {
        const int bi = key / p.block_size;
        int64_t blk = (key < kv_end && bi < p.max_blocks) ? bt[bi] : 0;
        if (blk < 0 || blk >= p.num_blocks) blk = 0;
        return ((blk * 2) * p.Hkv + kvh) * p.block_size + (key % p.block_size);
      };
      auto load_k = [&](int i) -> bool {
        const int stage = i & 1;
        if (i >= kStages && !wait_or_abort(&k_empty[stage], ((i >> 1) - 1) & 1, ab, 801)) return false;
        mbar_expect_tx(&k_full[stage], kKBytes);
        uint8_t* sK = smem + stage * kKBytes;
#pragma unroll
        for (int pg = 0; pg < kKTile / kPage; ++pg) {
          const int key = kv_begin + i * kKTile + pg * kPage;
          uint8_t* dst = sK + pg * (kPage * 128);
          if constexpr (kMla) {
            // rows past the request's keys belong to the next request or lie outside the tensor (zero fill): masked
#pragma unroll
            for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * kHalfBytes, &tmKV, &k_full[stage], head * 256 + h * 64, kv_row0 + key);
            tma_load_2d(dst + 2 * kHalfBytes, &tmKpe, &k_full[stage], 0, kv_row0 + key);
          } else {
            const int64_t rowK = page_row(key);
#pragma unroll
            for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * kHalfBytes, &tmKV, &k_full[stage], h * 64, (int)rowK);
          }
        }
        return true;
      };
      auto load_v = [&](int i) -> bool {
        const int stage = i % kVStages, use = i / kVStages;
        if (i >= kVStages && !wait_or_abort(&v_empty[stage], (use - 1) & 1, ab, 804)) return false;
        mbar_expect_tx(&v_full[stage], kOpBytes);
        uint8_t* sV = sVr + stage * kOpBytes;
#pragma unroll
        for (int pg = 0; pg < kKTile / kPage; ++pg) {
          const int key = kv_begin + i * kKTile + pg * kPage;
          uint8_t* dst = sV + pg * (kPage * 128);
          if constexpr (kMla) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_2d(dst + h * kHalfBytes, &tmKV, &v_full[stage], head * 256 + 128 + h * 64, kv_row0 + key);
          } else {
            const int64_t rowV = page_row(key) + (int64_t)p.Hkv * p.block_size;
#pragma unroll
            for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * kHalfBytes, &tmKV, &v_full[stage], h * 64, (int)rowV);
          }
        }
        return true;
      };
      // order: K of the next tile before V of this one, so that S(i + 1) never waits behind the V ring
      int issued_k = 0, issued_v = 0;
      bool ok = true;
      for (int j = 0; ok && j <= n_tiles; ++j) {      // K(0), K(1), V(0), K(2), V(1), ...
        if (j < n_tiles) {
          ok = load_k(j);
          if (ok) ++issued_k;
        }
        if (ok && j >= 1) {
          ok = load_v(j - 1);
          if (ok) ++issued_v;
        }
      }
      if (!ok) {   // let the copies in flight land before the CTA's shared memory goes away (bounded)
        for (int i = max(0, issued_k - kStages); i < issued_k; ++i)
          for (uint32_t q2 = 0; q2 < (1u << 16); ++q2)
            if (mbar_try_wait(&k_full[i & 1], (i >> 1) & 1)) break;
        for (int i = max(0, issued_v - kVStages); i < issued_v; ++i)
          for (uint32_t q2 = 0; q2 < (1u << 16); ++q2)
            if (mbar_try_wait(&v_full[i % kVStages], (i / kVStages) & 1)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (event-driven)
    if (elect_one() && n_tiles > 0) {
      const uint32_t fmt = FmtOf<T>::v;
      const uint32_t idesc_s = umma_idesc(kQTile, kKTile, fmt, fmt, 0, 0);   // A = Q, B = K tile, both K-major
      const uint32_t idesc_o = umma_idesc(kQTile, kD, fmt, fmt, 0, 1);       // A = P (K-major), B = V tile (MN-major)
      const uint32_t tS = tmem_base, tO = tmem_base + 2 * kKTile;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int i) {
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + (i & 1) * kKBytes);
#pragma unroll
        for (int k = 0; k < kQBlocks * 4; ++k) {
          const int kb = k / 4, kk = k % 4;
          umma_f16(tS + (i & 1) * kKTile, umma_desc_k_sw128(q_addr + kb * kHalfBytes + kk * 32),
                   umma_desc_k_sw128(k_addr + kb * kHalfBytes + kk * 32), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[i & 1]);
        umma_commit(&k_empty[i & 1]);
        if (i == 5) trace_mark(p.trace, cta_id, 13);
      };
      auto issue_pv = [&](int i) {
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sVr + (i % kVStages) * kOpBytes);
#pragma unroll
        for (int k = 0; k < kKTile / 16; ++k) {
          // A: 16 keys of P (key block k / 4, 32 bytes in); B: the same 16 keys of V, 128 dims (two 64-dim blocks)
          umma_f16(tO, umma_desc_k_sw128(p_addr + (k / 4) * kHalfBytes + (k % 4) * 32),
                   umma_desc_mn_sw128(v_addr + k * 2048, kHalfBytes, 1024), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        }
        if (i == 3) trace_mark(p.trace, cta_id, 12);
        umma_commit(o_done);   // first: whoever has seen p_free of this tile may rely on o_done having advanced
        umma_commit(&v_empty[i % kVStages]);
        umma_commit(p_free);
        if (i == n_tiles - 1) umma_commit(o_final);
      };
      bool ok = wait_or_abort(q_full, 0, ab, 802);
      int next_s = 0, next_pv = 0;
      uint32_t spins = 0;
      while (ok && next_pv < n_tiles) {
        bool progressed = false;
        if (next_s < n_tiles && next_s <= next_pv + 1 && mbar_try_wait(&k_full[next_s & 1], (next_s >> 1) & 1) &&
            (next_s < 2 || mbar_try_wait(&s_empty[next_s & 1], ((next_s >> 1) - 1) & 1))) {
          issue_s(next_s);
          ++next_s;
          progressed = true;
        }
        if (next_pv < next_s && mbar_try_wait(p_ready, next_pv & 1) &&
            mbar_try_wait(&v_full[next_pv % kVStages], (next_pv / kVStages) & 1)) {
          if (next_pv == 4) trace_mark(p.trace, cta_id, 9);
          issue_pv(next_pv);
          ++next_pv;
          progressed = true;
        }
        if (progressed) { spins = 0; continue; }
        if (++spins > (1u << 20)) { ab.raise(803); break; }
        if ((spins & 255) == 255 && ab.aborted()) break;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                 // row of the tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_off, tO = tmem_base + 2 * kKTile + lane_off;
    const bool row_ok = r < n_rows;
    const int pos = ctx + row0 + r;                    // position of this row's token
    float m_used = -INFINITY, l_sum = 0.f;
    bool fail = false;
    for (int i = 0; i < n_tiles; ++i) {
      const int buf = i & 1;
      if (!fail && !wait_or_abort(&s_full[buf], (i >> 1) & 1, ab, 805)) fail = true;
      tc_fence_after_sync();
      if (threadIdx.x == 64 && i == 0) trace_mark(p.trace, cta_id, 1);
      if (threadIdx.x == 64 && i == 4) trace_mark(p.trace, cta_id, 2);
      if (threadIdx.x == 64 && i == 5) trace_mark(p.trace, cta_id, 7);
      if (threadIdx.x == 64 && i == 20) trace_mark(p.trace, cta_id, 8);
      const int key0 = kv_begin + i * kKTile;
      const bool full_tile = key0 + kKTile - 1 <= pos_first && key0 + kKTile <= kv_end &&
                             (p.window <= 0 || key0 > pos_last - p.window);
      // ---- the whole row (128 scores) in one TMEM round trip: a tcgen05.ld + wait pair costs several hundred
      // nanoseconds whatever its width, so all four 32-column loads are issued before the single wait, and the
      // S buffer goes back to the tensor core at once
      uint32_t v[kKTile];
#pragma unroll
      for (int c = 0; c < kKTile; c += 32) tmem_ld_x32_p(tS + buf * kKTile + c, v + c);
      tmem_ld_wait();
      if (threadIdx.x == 64 && i == 4) trace_mark(p.trace, cta_id, 11);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);
      // One warp per scheduler: nothing hides instruction latency but independent work inside the thread, so the
      // row maximum runs on four partial maxima and the exponentials in chunks of 32 with four partial sums; the
      // raw scores are masked in place and scaled inside the exponent (one FMA + one ex2 per element).
      if (!full_tile) {
#pragma unroll
        for (int e = 0; e < kKTile; ++e) {
          const int key = key0 + e;
          const bool in = key < kv_end && key <= pos && (p.window <= 0 || key > pos - p.window);
          v[e] = in ? v[e] : 0xff800000u;   // -inf
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < kKTile; e += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], __uint_as_float(v[e + u]));
      }
      float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // scale > 0: max commutes
      if (!row_ok) tmax = -INFINITY;
      if (threadIdx.x == 64 && i == 4) trace_mark(p.trace, cta_id, 3);
      // ---- lazy running maximum; the rescale of O is warp-collective (TMEM access), so the warp decides together
      float alpha = 1.f;
      const bool bump = tmax > m_used + kMaxSlack;
      if (bump) { alpha = exp2f(m_used - tmax); m_used = tmax; l_sum *= alpha; }
      // P (one buffer): the previous P.V must have read it (it has, long ago, unless the tensor pipe is behind);
      // this also keeps o_done within one phase
      if (i >= 1 && !fail && !wait_or_abort(p_free, (i - 1) & 1, ab, 806)) fail = true;
      if (threadIdx.x == 64 && i == 4) trace_mark(p.trace, cta_id, 4);
      if (__any_sync(0xffffffffu, bump) && i > 0) {
        if (!fail && !wait_or_abort(o_done, (i - 1) & 1, ab, 808)) fail = true;
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < kD; c += 32) {   // rare path: 32 columns at a time keeps the register count down
          uint32_t o[32];
          tmem_ld_x32_p(tO + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st_x32_p(tO + c, o);
        }
        tmem_st_wait();
      }
      // ---- exponentials, row sum and the P row (16-bit, K-major over keys, 16-byte chunks swizzled by row; keys
      // 8 q .. 8 q + 7 = chunk q % 8 of key block q / 8), 32 keys at a time
      const float neg_ms = (m_used == -INFINITY || !row_ok) ? -INFINITY : -m_used;   // invalid rows: P = 0
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kKTile; c += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float pe[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            pe[u] = ex2_approx(fmaf(__uint_as_float(v[c + e + u]), p.scale_log2, neg_ms));
            ls[u] += pe[u];
          }
          pk[e / 2] = pack2<T>(pe[0], pe[1]);
          pk[e / 2 + 1] = pack2<T>(pe[2], pe[3]);
        }
        if (!fail) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int q = c / 8 + q4;
            *reinterpret_cast<uint4*>(sP + (q >> 3) * kHalfBytes + r * 128 + (((q & 7) ^ (r & 7)) << 4)) =
                make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
          }
        }
      }
      l_sum += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      const bool warp_failed = __any_sync(0xffffffffu, fail);
      __syncwarp();
      if (lane == 0 && !warp_failed) mbar_arrive(p_ready);
      if (threadIdx.x == 64 && i == 4) trace_mark(p.trace, cta_id, 5);
    }
    if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 6);
    // ---- epilogue
    bool ok = !fail;
    if (ok && n_tiles > 0) {
      if (!wait_or_abort(o_final, 0, ab, 807)) ok = false;
      tc_fence_after_sync();
    }
    if (n_tiles > 0) {
      const int64_t orow = (int64_t)(qs + row0 + r) * p.Hq + head;
      float den = l_sum;
      const float ms = (m_used == -INFINITY) ? 0.f : m_used;
      if (p.sinks != nullptr) den += exp2f(p.sinks[head] * 1.4426950408889634f - ms);
      const float inv = (ok && den > 0.f) ? 1.f / den : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + orow * kD;
      uint32_t o[kD];
#pragma unroll
      for (int c = 0; c < kD; c += 32) tmem_ld_x32_p(tO + c, o + c);   // warp-collective: every lane loads
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < kD / 8; ++q4) {
          uint32_t w4[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            w4[u] = pack2<T>(__uint_as_float(o[q4 * 8 + 2 * u]) * inv, __uint_as_float(o[q4 * 8 + 2 * u + 1]) * inv);
          *reinterpret_cast<uint4*>(dst + q4 * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
      }
      if (row_ok && p.lse != nullptr) p.lse[orow] = (ok && den > 0.f) ? (ms + log2f(den)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 64) trace_mark(p.trace, cta_id, 10);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, bool kMla>
static int launch(const Params& p, const CUtensorMap& tmQ, const CUtensorMap& tmKV, const CUtensorMap& tmKpe, int B,
                  int max_query_len, cudaStream_t st) {
  auto kern = prefill_umma_kernel<T, kMla>;
  const size_t smem = Cfg<kMla>::kSmem;
  cudaError_t e = ensure_dynamic_smem((const void*)kern, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((unsigned)((max_query_len + kQTile - 1) / kQTile), (unsigned)p.Hq, (unsigned)B);
  return (int)launch_pdl(kern, grid, dim3(kThreads), smem, st, tmQ, tmKV, tmKpe, p);
}

}  // namespace pattn
}  // namespace b200

// Paged GQA prefill attention on tcgen05 (head_dim 128, block_size a multiple of 64).  `tmQ`: q as a 2-D
// [T, Hq * 128] 16-bit tensor with 64-column x 128-row boxes; `tmKV`: the cache as [rows, 128] with 64 x 64 boxes;
// both with 128-byte swizzle.  Returns 3 for shapes it does not serve.
extern "C" int b200_prefill_attention_umma(void* out, float* lse, const void* tmQ, const void* tmKV,
                                           const int* block_tables, const int* seq_lens, const int* qsl,
                                           const float* sinks, int* status, int B, int Hq, int Hkv, int D, int block_size,
                                           int max_blocks, int64_t num_blocks, int max_query_len, int window, float scale,
                                           int dtype, unsigned long long* trace, cudaStream_t st) {
  using namespace b200;
  if (B == 0 || max_query_len <= 0) return 0;
  if (D != 128 || Hq % Hkv || block_size % pattn::kPage || B > 65535 || Hq > 65535) return 3;
  pattn::Params p;
  p.out = out; p.lse = lse; p.block_tables = block_tables; p.seq_lens = seq_lens; p.qsl = qsl; p.sinks = sinks;
  p.status = status; p.trace = trace; p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size; p.max_blocks = max_blocks; p.window = window;
  p.num_blocks = num_blocks; p.scale_log2 = scale * 1.4426950408889634f;
  p.kv_starts = nullptr; p.causal = 1;
  const CUtensorMap& q = *reinterpret_cast<const CUtensorMap*>(tmQ);
  const CUtensorMap& kv = *reinterpret_cast<const CUtensorMap*>(tmKV);
  if (dtype == 1) return pattn::launch<__nv_bfloat16, false>(p, q, kv, kv, B, max_query_len, st);
  if (dtype == 2) return pattn::launch<__half, false>(p, q, kv, kv, B, max_query_len, st);
  return 3;
}

// Multi-head latent attention prefill in the compute-friendly form (192-dim q / k, 128-dim v) on tcgen05.
// `tmQ`: q as [T, Hq * 192] with 64-column x 128-row boxes; `tmKV`: the up-projected keys / values as
// [rows, Hq * 256] (k_nope | v per head) with 64 x 64 boxes; `tmKpe`: the rotary keys as [rows, 64] with 64 x 64
// boxes; all 16-bit with 128-byte swizzle and row extents equal to the number of valid rows.  Request r owns key rows
// kv_starts[r] .. kv_starts[r] + kv_lens[r] and query rows qsl[r] .. qsl[r + 1]; causal: its queries are its last
// keys.  Rows of requests with no key are not written (the caller presets out = 0, lse = -inf).
extern "C" int b200_mla_prefill_umma(void* out, float* lse, const void* tmQ, const void* tmKV, const void* tmKpe,
                                     const int* kv_starts, const int* kv_lens, const int* qsl, int* status, int B,
                                     int Hq, int max_query_len, int causal, float scale, int dtype,
                                     unsigned long long* trace, cudaStream_t st) {
  using namespace b200;
  if (B == 0 || max_query_len <= 0) return 0;
  if (B > 65535 || Hq > 65535) return 3;
  pattn::Params p;
  p.out = out; p.lse = lse; p.block_tables = nullptr; p.seq_lens = kv_lens; p.qsl = qsl; p.kv_starts = kv_starts;
  p.sinks = nullptr; p.status = status; p.trace = trace; p.Hq = Hq; p.Hkv = Hq; p.block_size = pattn::kPage;
  p.max_blocks = 0; p.window = 0; p.causal = causal ? 1 : 0; p.num_blocks = 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  const CUtensorMap& q = *reinterpret_cast<const CUtensorMap*>(tmQ);
  const CUtensorMap& kv = *reinterpret_cast<const CUtensorMap*>(tmKV);
  const CUtensorMap& kpe = *reinterpret_cast<const CUtensorMap*>(tmKpe);
  if (dtype == 1) return pattn::launch<__nv_bfloat16, true>(p, q, kv, kpe, B, max_query_len, st);
  if (dtype == 2) return pattn::launch<__half, true>(p, q, kv, kpe, B, max_query_len, st);
  return 3;
}
