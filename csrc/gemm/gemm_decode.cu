// Decode-sized bf16/fp16 GEMM for sm_100a:  out[T <= 32, N] = x[T, K] . W[N, K]^T (+ bias), one token tile.
//
// A decode step is a chain of small dependent kernels, so what counts is how short the dependent
// latency chain inside each kernel is and how many SMs pull weight bytes at the same time.  This
// kernel therefore
//   * gives every 128-row weight tile to a thread-block CLUSTER of S CTAs (1 <= S <= 8) that split the
//     K range; the partial accumulators meet in the leader CTA's shared memory (st.shared::cluster +
//     a remote mbarrier arrive), not in a global workspace with a fence, an atomic ticket and a re-read;
//     the leader sums the partials in rank order, so the result is deterministic;
//   * runs one tile per CTA (no persistent loop): with two CTAs resident per SM all CTAs of a
//     weight matrix stream concurrently and share HBM bandwidth evenly, whatever the tile count;
//   * streams its first weight tiles before waiting for the previous kernel (programmatic dependent
//     launch), like the general kernel in gemm_bf16.cu;
//   * finishes with one of several epilogues on the leader: plain (+ bias), gated activation over
//     [64 gate | 64 up] interleaved weight tiles, or the row-parallel form under tensor parallelism:
//     store the local partial AND push it, as {2 x 16-bit, epoch} 8-byte units, straight into every
//     peer's low-latency all-reduce slot over NVLink (plain peer stores), so that the kernel after it
//     only collects, adds the residual and normalises (all-reduce call sites C1 / C2 of the reference,
//     vllm_kunlun/models/deepseek_v2.py:126-134,399-405).
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 TMEM owner + tcgen05.mma issuer, warps 2-5 epilogue.
// TMA loads carry no cluster multicast.  Every wait is bounded; on time-out the status word is set and the
// CTA unwinds (drains its copies, meets the cluster barrier, frees TMEM).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "gemm_common.cuh"

namespace b200 {

namespace dec {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kThreadsW4 = 320;   // 4-bit weights: four more warps de-quantise
constexpr int kStageBytesA = BM * BK * 2;
constexpr int kTileStride = BM + 8;  // staging row (elements of OutT)

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float gated(float g, float u, int act) {
  if (act == 1) return g / (1.f + __expf(-g)) * u;
  if (act == 2) {
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * g * (1.f + t) * u;
  }
  g = fminf(g, 7.f);
  u = fminf(fmaxf(u, -7.f), 7.f);
  return g / (1.f + __expf(-1.702f * g)) * (u + 1.f);
}

// Low-latency all-reduce slots of every rank (peer mappings); see comm/allreduce.cu for the layout.
struct Comm {
  void* ll_bufs[8];
  const uint32_t* epoch_word;
  int64_t slot_bytes;
  int on, rank, nranks;
};

// qkv epilogue: weight tile nt is exactly head nt (head_dim 128 = BM), so per-head q / k RMSNorm, the rotary embedding
// and the K / V scatter into the paged cache are tile-local and run in the leader CTA's epilogue instead of in a
// kernel of their own (the reference chains `_C::split_norm_rope_neox` and `reshape_and_cache_flash`,
// ops/_kunlun_ops.py; the stand-alone form here is qkv_split_norm_rope_cache_kernel in cache_rope.cu).
struct QkvEpi {
  const int64_t* positions;   // [T]
  const float* cos_sin;       // [max_pos][128]: cos (64) | sin (64)
  const void* q_w;            // [128] or null
  const void* k_w;            // [128] or null
  void* kv_cache;             // [blocks][2][Hkv][block_size][128]
  const int64_t* slots;       // [T]
  int64_t num_blocks, max_pos;
  float eps;
  int on, Hq, Hkv, neox, gemma, block_size;
};

constexpr int kAccBufs = 4;  // fp8: accumulator buffers handed to the epilogue one k-block at a time

// 4-bit weights: the TMA ring then carries, per k-block, the activation tile and the PACKED weight tile (128 rows x
// 32 bytes) - 6 or 8 KB a stage, so the ring is deep enough to keep HBM busy - and the 16-bit A tiles live in a ring
// of their own (kW4Tiles x 16 KB): the four epilogue warps (one thread per weight row), idle during the main loop
// otherwise, turn each packed tile into a 128-byte-swizzled A tile and hand it to the MMA issuer through `deq_bar`;
// the tensor core's commit frees the A tile (`afree_bar`) and the ring stage.
constexpr int kPackedBytes = BM * (BK / 2);
constexpr int kW4Tiles = 3;
struct W4 {
  const void* scale;   // [N, K / group], activation type
  const void* zero;    // [N, K / group], activation type (integer-valued)
  int group, on;
};

// Eight 4-bit values of a packed word -> four pairs of 16-bit floats (q - zero) * scale.  The nibbles of a word are
// stored in the order 0, 2, 4, 6, 1, 3, 5, 7 of its eight consecutive k positions, so that `(w >> 4 j) & 0x000F000F`
// is the pair (2 j, 2 j + 1); or-ing the exponent of 128 (bf16) / 1024 (fp16) makes each half the exact value
// 128 + q / 1024 + q, and one subtraction of (128 + zero) and one multiplication finish the job - the same value
// as rounding (q - zero) * scale once from fp32.
template <typename OutT> struct W4Cvt;
template <> struct W4Cvt<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;
  static constexpr float kBase = 128.f;
};
template <> struct W4Cvt<__half> {
  using V2 = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;
  static constexpr float kBase = 1024.f;
};
template <typename OutT>
__device__ __forceinline__ uint4 w4_convert(uint32_t w, typename W4Cvt<OutT>::V2 off, typename W4Cvt<OutT>::V2 sc) {
  using V2 = typename W4Cvt<OutT>::V2;
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | W4Cvt<OutT>::kMagic;
    V2 v = __hmul2(__hsub2(*reinterpret_cast<V2*>(&t), off), sc);
    r[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

template <int BN>
struct Cfg {
  static constexpr int kStageBytes = kStageBytesA + BN * BK * 2;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static constexpr int kTmemColsFp8 = kAccBufs * BN;                // 64 or 128
  static constexpr int kSlotBytes = BN * BM * 4;                    // one partial tile: [BN / 4][128 features] float4
  static constexpr int kTileBytes = BN * kTileStride * 2;
};

// kFp8: e4m3 operands with 128x128 weight block scales (w_scale [ceil(N/128)][ceil(K/128)]) and 1x128 activation
// scales (a_scale [ceil(K/128)][a_stride], transposed).  A k-block is then 128 K-elements (still one 128-byte
// swizzle row per operand row); every k-block is accumulated by the tensor core into its own TMEM buffer and the
// epilogue warps multiply it by a_scale[kb][t] * w_scale[nt][kb] while adding it into fp32 registers, overlapped
// with the next k-block's MMAs.
template <int BN, typename OutT, bool kFp8>
__global__ void __launch_bounds__(kThreadsW4)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   OutT* __restrict__ out, const OutT* __restrict__ bias, int* __restrict__ status, int T, int N, int K,
                   int kb_per_cta, int fmt, int ldo, int num_stages, int S, int act, int l2_prefetch,
                   const float* __restrict__ a_scale, const float* __restrict__ w_scale, int a_stride,
                   const __grid_constant__ Comm cm, const __grid_constant__ QkvEpi qk, const __grid_constant__ W4 w4p) {
  using C = Cfg<BN>;
  constexpr int BKE8 = 128;             // K elements per k-block of 8-bit operands (still one 128-byte swizzle row)
  // fmt == 2 (non-fp8 instantiation): signed 8-bit operands on kind::i8 with per-token activation scales
  // (a_scale [T]) and per-channel weight scales (w_scale [N]) applied by the final epilogue
  const bool i8 = !kFp8 && fmt == 2;
  const int BKE = (kFp8 || i8) ? BKE8 : BK;  // K elements per k-block
  const bool w4 = !kFp8 && w4p.on != 0;      // 4-bit weights, de-quantised into the stage's A tile by the epilogue warps
  const int stage_bytes = w4 ? BN * BK * 2 + kPackedBytes : C::kStageBytes;   // 4-bit: [x tile | packed weight tile]
  const uint32_t stage_tx = (uint32_t)stage_bytes;
  constexpr int kCols = kFp8 ? C::kTmemColsFp8 : C::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem_al = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_ring = smem_al;                                             // 4-bit: kW4Tiles de-quantised A tiles
  uint8_t* smem = smem_al + (w4 ? kW4Tiles * kStageBytesA : 0);          // the TMA ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + num_stages * stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + num_stages;
  uint64_t* tmem_full = bars + 2 * num_stages;
  uint64_t* red_bar = tmem_full + 1;
  uint64_t* acc_full = red_bar + 1;             // [kAccBufs] (fp8)
  uint64_t* acc_empty = acc_full + kAccBufs;    // [kAccBufs] (fp8)
  uint64_t* deq_bar = acc_empty + kAccBufs;     // [kW4Tiles] (4-bit weights): 4 arrivals, one per epilogue warp
  uint64_t* afree_bar = deq_bar + 4;            // [kW4Tiles] the MMAs that read the A tile are complete
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(deq_bar + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  volatile int* ep_ok_slot = reinterpret_cast<volatile int*>(tmem_base_slot + 2);  // [2]
  uint8_t* after = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tmem_base_slot + 4) + 15) & ~uintptr_t(15));
  float4* slots = reinterpret_cast<float4*>(after);                                 // [(S-1)][BN / 4][128]
  OutT* tile = reinterpret_cast<OutT*>(after + (size_t)(S - 1) * C::kSlotBytes);    // [BN][128 + 8]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = (S > 1) ? cluster_ctarank() : 0u;
  const int nt = blockIdx.x / S;
  const int total_kb = (K + BKE - 1) / BKE;
  const int kb0 = (int)crank * kb_per_cta;
  const int kb1 = min(total_kb, kb0 + kb_per_cta);
  const int nkb = kb1 - kb0;  // >= 1 by construction on the host
  Abort ab{status, abort_flag};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < kW4Tiles; ++b) { mbar_init(&deq_bar[b], 4); mbar_init(&afree_bar[b], 1); }
    mbar_init(tmem_full, 1);
    mbar_init(red_bar, (uint32_t)(S > 1 ? (S - 1) * 4 : 1));
    for (int b = 0; b < kAccBufs; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_fence_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
    griddep_launch();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (S > 1) {  // the leader's reduction barrier must exist before any peer CTA can arrive on it
    cluster_arrive();
    cluster_wait();
  }
  const uint32_t tmem_base = *tmem_base_slot;

  // ---- 4-bit weights: a group of four warps (one thread per weight row) turns the packed tile of every ndg-th k-block
  // into a 16-bit A tile (128-byte swizzle).  Group 0 = the epilogue warps, group 1 = warps 6 - 9 when the block was
  // launched with 320 threads; the groups alternate over the k-blocks.
  const int ndg = (int)(blockDim.x - 64) / 128;
  auto dequant_rows = [&](int grp, int n_local) {
    using V2 = typename W4Cvt<OutT>::V2;
    const int row = nt * BM + n_local;
    const int groups = K / w4p.group;                         // scale / zero row length
    const OutT* sc_row = reinterpret_cast<const OutT*>(w4p.scale) + (size_t)row * groups;
    const OutT* zr_row = reinterpret_cast<const OutT*>(w4p.zero) + (size_t)row * groups;
    const bool row_in = row < N;
    const int kpg = w4p.group / BK;                           // k-blocks per quantisation group
    const int kshift = (kpg & (kpg - 1)) == 0 ? __ffs(kpg) - 1 : -1;
    auto group_of = [&](int kb) { return kshift >= 0 ? (kb >> kshift) : kb / kpg; };
    uint32_t coff[8];                                         // swizzled position of 16-byte chunk j of this row
#pragma unroll
    for (int j = 0; j < 8; ++j) coff[j] = (uint32_t)((j ^ (n_local & 7)) << 4);
    const uint8_t* pk_base = smem + BN * BK * 2 + n_local * (BK / 2);
    uint8_t* a_base = a_ring + n_local * 128;
    int stage = grp % num_stages, slot = grp % kW4Tiles;
    uint32_t phase = (uint32_t)((grp / num_stages) & 1), sph = (uint32_t)((grp / kW4Tiles) & 1);
    // group parameters are fetched one step ahead: no dependent global load in front of the conversion
    int g_cur = -1, g_nxt = group_of(kb0 + grp);
    OutT s_nxt = from_float<OutT>(0.f), z_nxt = from_float<OutT>(0.f);
    if (row_in && grp < nkb) { s_nxt = sc_row[g_nxt]; z_nxt = zr_row[g_nxt]; }
    V2 off = V2(s_nxt, s_nxt), sc = off;
    for (int i = grp; i < nkb; i += ndg) {
      const int gi = g_nxt;
      if (gi != g_cur) {
        g_cur = gi;
        const OutT o1 = from_float<OutT>(W4Cvt<OutT>::kBase + to_float<OutT>(z_nxt));
        sc = V2(s_nxt, s_nxt);
        off = V2(o1, o1);
      }
      if (i + ndg < nkb) {
        g_nxt = group_of(kb0 + i + ndg);
        if (g_nxt != gi && row_in) { s_nxt = sc_row[g_nxt]; z_nxt = zr_row[g_nxt]; }
      }
      // every warp waits by itself (lane 0 with the bound, the others once the phase is known to be complete)
      int ok_w = 1;
      if (lane == 0) {
        ok_w = (i < kW4Tiles || wait_or_abort(&afree_bar[slot], sph ^ 1u, ab, 130)) &&
               wait_or_abort(&full_bar[stage], phase, ab, 128);
      }
      ok_w = __shfl_sync(0xffffffffu, ok_w, 0);
      if (!ok_w) break;
      while (!mbar_try_wait(&full_bar[stage], phase)) {}
      if (i >= kW4Tiles) { while (!mbar_try_wait(&afree_bar[slot], sph ^ 1u)) {} }
      tc_fence_after_sync();
      const uint4* pk = reinterpret_cast<const uint4*>(pk_base + stage * stage_bytes);
      const uint4 p0 = pk[0], p1 = pk[1];
      const uint32_t wds[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      uint8_t* arow = a_base + slot * kStageBytesA;
#pragma unroll
      for (int j = 0; j < 8; ++j)   // word j = k positions 8 j .. 8 j + 7 = 16-byte chunk j of the row
        *reinterpret_cast<uint4*>(arow + coff[j]) = w4_convert<OutT>(wds[j], off, sc);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&deq_bar[slot]);
      stage += ndg;
      if (stage >= num_stages) { stage -= num_stages; phase ^= 1u; }
      slot += ndg;
      if (slot >= kW4Tiles) { slot -= kW4Tiles; sph ^= 1u; }
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      int pre = 0;
      // weights do not depend on the previous kernel: fill the ring (and pull what follows into L2) first
      for (; pre < num_stages && pre < nkb; ++pre) {
        mbar_expect_tx(&full_bar[pre], stage_tx);
        if (w4) tma_load_2d_hint(smem + pre * stage_bytes + BN * BK * 2, &tmW, &full_bar[pre], (kb0 + pre) * (BK / 2), nt * BM, pol_w);
        else tma_load_2d_hint(smem + pre * stage_bytes, &tmW, &full_bar[pre], (kb0 + pre) * BKE, nt * BM, pol_w);
      }
      for (int i = 0; i < l2_prefetch && pre + i < nkb && !w4; ++i) tma_prefetch_l2_2d(&tmW, (kb0 + pre + i) * BKE, nt * BM);
      griddep_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < nkb; ++i) {
        uint8_t* sa = smem + stage * stage_bytes;
        uint8_t* sb = w4 ? sa : sa + kStageBytesA;
        if (i < pre) {
          tma_load_2d(sb, &tmX, &full_bar[stage], (kb0 + i) * BKE, 0);
        } else {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1, ab, 121)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], stage_tx);
          if (w4) tma_load_2d_hint(sa + BN * BK * 2, &tmW, &full_bar[stage], (kb0 + i) * (BK / 2), nt * BM, pol_w);
          else tma_load_2d_hint(sa, &tmW, &full_bar[stage], (kb0 + i) * BKE, nt * BM, pol_w);
          tma_load_2d(sb, &tmX, &full_bar[stage], (kb0 + i) * BKE, 0);
        }
        ++issued;
        if (++stage == num_stages) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        int pending = issued < num_stages ? issued : num_stages;
        for (int i = 0; i < pending; ++i) {
          int s = (stage - 1 - i + 2 * num_stages) % num_stages;
          uint32_t ph = (s < stage) ? phase : (phase ^ 1);
          for (uint32_t p = 0; p < (1u << 16); ++p)
            if (mbar_try_wait(&full_bar[s], ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      // the first full barrier needs the activations, i.e. the previous kernel: wait for that dependency here
      // (unbounded by nature) so that the bounded wait below covers only the copies
      griddep_wait();
      const uint32_t idesc = kFp8 ? umma_idesc(BM, BN, 0, 0) : (i8 ? umma_idesc_i8(BM, BN) : umma_idesc(BM, BN, fmt, fmt));
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        if (!wait_or_abort(&full_bar[stage], phase, ab, 123)) { ok = false; break; }
        if (w4 && !wait_or_abort(&deq_bar[i % kW4Tiles], (i / kW4Tiles) & 1, ab, 129)) { ok = false; break; }
        const int ab_buf = i % kAccBufs;
        if (kFp8 && i >= kAccBufs && !wait_or_abort(&acc_empty[ab_buf], ((i / kAccBufs) - 1) & 1, ab, 126)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t sa = smem_u32(smem + stage * stage_bytes);
        uint32_t sb = sa + kStageBytesA;
        if (w4) {
          sb = sa;
          sa = smem_u32(a_ring + (i % kW4Tiles) * kStageBytesA);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte row: 16 16-bit or 32 8-bit elements each
          uint64_t da = umma_desc_k_sw128(sa + k * 32);
          uint64_t db = umma_desc_k_sw128(sb + k * 32);
          if (kFp8) umma_f8(tmem_base + ab_buf * BN, da, db, idesc, k > 0 ? 1u : 0u);
          else if (i8) umma_i8(tmem_base, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
          else umma_f16(tmem_base, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (w4) umma_commit(&afree_bar[i % kW4Tiles]);
        if (kFp8) umma_commit(&acc_full[ab_buf]);
        if (++stage == num_stages) { stage = 0; phase ^= 1; }
      }
      if (ok && !kFp8) umma_commit(tmem_full);
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ second de-quantising group (4-bit weights)
    griddep_wait();
    if (w4) dequant_rows(1, (warp - 6) * 32 + lane);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int ep_tid = (warp - 2) * 32 + lane;
    const int n_local = quarter * 32 + lane;
    griddep_wait();
    if (w4) dequant_rows(0, n_local);
    float acc[BN];
    bool acc_ok = true;
    if (kFp8) {
#pragma unroll
      for (int c = 0; c < BN; ++c) acc[c] = 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const int wkb = total_kb;  // w_scale row length
      // the scales of a k-block are fetched one k-block ahead: no dependent global load in front of the FMAs
      float ws_next = w_scale[(size_t)nt * wkb + kb0];
      float as_next[BN];
#pragma unroll
      for (int c = 0; c < BN; ++c) as_next[c] = (c < T) ? __ldg(a_scale + (size_t)kb0 * a_stride + c) : 0.f;
      for (int i = 0; i < nkb; ++i) {
        const int buf = i % kAccBufs;
        float sc[BN];
#pragma unroll
        for (int c = 0; c < BN; ++c) sc[c] = as_next[c] * ws_next;
        if (i + 1 < nkb) {
          ws_next = w_scale[(size_t)nt * wkb + kb0 + i + 1];
#pragma unroll
          for (int c = 0; c < BN; ++c) as_next[c] = (c < T) ? __ldg(a_scale + (size_t)(kb0 + i + 1) * a_stride + c) : 0.f;
        }
        if (ep_tid == 0) ep_ok_slot[i & 1] = wait_or_abort(&acc_full[buf], (i / kAccBufs) & 1, ab, 127) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_ok_slot[i & 1] == 0) { acc_ok = false; break; }
        while (!mbar_try_wait(&acc_full[buf], (i / kAccBufs) & 1)) {}
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + buf * BN + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), sc[c + j], acc[c + j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
    } else {
      if (ep_tid == 0) ep_ok_slot[0] = wait_or_abort(tmem_full, 0, ab, 124) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      acc_ok = ep_ok_slot[0] != 0;
    }
    if (kFp8) {
      // accumulated above
    } else if (acc_ok) {
      while (!mbar_try_wait(tmem_full, 0)) {}
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        tmem_ld_x16(taddr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c + j] = i8 ? (float)(int)r[j] : __uint_as_float(r[j]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < BN; ++c) acc[c] = 0.f;
    }
    if (S > 1 && crank != 0) {
      // partial tile -> the leader's slot [crank - 1][token / 4][feature] (16 bytes per lane, lane-contiguous),
      // then one arrival per warp
      const uint32_t local = smem_u32(slots + (size_t)(crank - 1) * (BN / 4) * BM + n_local);
      const uint32_t remote = mapa(local, 0);
#pragma unroll
      for (int c = 0; c < BN; c += 4)
        st_cluster_v4(remote + (c / 4) * BM * 16, acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
      fence_acq_rel_cluster();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa(smem_u32(red_bar), 0));
    } else {
      bool ok = acc_ok;
      if (S > 1) {
        if (ep_tid == 0) {
          bool got = false;
          for (uint32_t i = 0; i < (1u << 22); ++i) {
            if (mbar_try_wait_cluster(red_bar, 0)) { got = true; break; }
            if ((i & 255) == 255 && ab.aborted()) break;
          }
          if (!got) ab.raise(125);
          ep_ok_slot[1] = got ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        ok = ok && ep_ok_slot[1] != 0;
        if (ok) {
          while (!mbar_try_wait_cluster(red_bar, 0)) {}
          for (int s = 0; s < S - 1; ++s) {  // rank order: deterministic
            const float4* src = slots + (size_t)s * (BN / 4) * BM + n_local;
#pragma unroll
            for (int c = 0; c < BN; c += 4) {
              float4 v = src[(c / 4) * BM];
              acc[c] += v.x; acc[c + 1] += v.y; acc[c + 2] += v.z; acc[c + 3] += v.w;
            }
          }
        }
      }
      if (ok) {
        // ---- final epilogue: stage [token][feature] as OutT, then 16-byte row segments
        const int n = nt * BM + n_local;
        const float bv = (bias != nullptr && n < N) ? to_float<OutT>(bias[n]) : 0.f;
        if (i8) {  // integer sums -> real values
          const float ws = n < N ? w_scale[n] : 0.f;
#pragma unroll
          for (int c = 0; c < BN; ++c) acc[c] *= ws * (c < T ? a_scale[c] : 0.f);
        }
#pragma unroll
        for (int c = 0; c < BN; ++c) tile[c * kTileStride + n_local] = from_float<OutT>(acc[c] + bv);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (qk.on) {
          // ---- head nt of the fused qkv row: warp = token (round-robin), lane = features l, l + 32, l + 64, l + 96 -
          // the same distribution (and so the same fp32 summation order) as the stand-alone kernel.  Values are read
          // back as OutT, i.e. rounded exactly as the stand-alone GEMM output would be.
          const int ew = warp - 2;
          const bool is_q = nt < qk.Hq, is_k = !is_q && nt < qk.Hq + qk.Hkv;
          const OutT* nw = reinterpret_cast<const OutT*>(is_q ? qk.q_w : (is_k ? qk.k_w : nullptr));
          float wv[4] = {1.f, 1.f, 1.f, 1.f};
          if (nw != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = to_float<OutT>(nw[lane + 32 * j]) + (qk.gemma ? 1.f : 0.f);
          }
          for (int rr = ew; rr < T; rr += 4) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = to_float<OutT>(tile[rr * kTileStride + lane + 32 * j]);
            if (is_q || is_k) {
              if (nw != nullptr) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) ss += v[j] * v[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float inv = rsqrtf(ss / 128 + qk.eps);
                // rounded to OutT between norm and rotary, as two separate kernels would
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = to_float<OutT>(from_float<OutT>(v[j] * inv * wv[j]));
              }
              int64_t pos = qk.positions[rr];
              pos = pos < 0 ? 0 : (pos >= qk.max_pos ? qk.max_pos - 1 : pos);
              const float* cs = qk.cos_sin + pos * 128;
              if (qk.neox) {  // pairs (d, d + 64) = (v[0], v[2]) and (v[1], v[3]) of this lane
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int f = lane + 32 * j;
                  const float c = cs[f], sn = cs[64 + f];
                  const float x0 = v[j], y0 = v[j + 2];
                  v[j] = x0 * c - y0 * sn;
                  v[j + 2] = y0 * c + x0 * sn;
                }
              } else {        // pairs (2 i, 2 i + 1): lanes l and l ^ 1
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int f = (lane + 32 * j) >> 1;
                  const float c = cs[f], sn = cs[64 + f];
                  const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                  v[j] = (lane & 1) == 0 ? v[j] * c - other * sn : v[j] * c + other * sn;
                }
              }
            }
            OutT* dst = nullptr;
            if (is_q) {
              dst = out + (size_t)rr * ldo + (size_t)nt * BM;
            } else if (qk.kv_cache != nullptr) {
              const int64_t slot = qk.slots[rr];
              if (slot >= 0 && slot < qk.num_blocks * qk.block_size) {
                const int kvh = is_k ? nt - qk.Hq : nt - qk.Hq - qk.Hkv;
                const int64_t blk = slot / qk.block_size, off = slot % qk.block_size;
                dst = reinterpret_cast<OutT*>(qk.kv_cache) +
                      ((((blk * 2 + (is_k ? 0 : 1)) * qk.Hkv + kvh) * qk.block_size + off) * (int64_t)BM);
              }
            }
            if (dst != nullptr) {
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = from_float<OutT>(v[j]);
            }
          }
        } else if (act != 0) {
          const int n0 = nt * (BM / 2);
          const int seg = ep_tid & 7;  // 8 segments of 8 output features
          for (int rr = ep_tid >> 3; rr < BN; rr += 16) {
            if (rr >= T) break;
            const OutT* gsrc = tile + rr * kTileStride + seg * 8;
            const OutT* usrc = gsrc + BM / 2;
            alignas(16) OutT res[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              res[e] = from_float<OutT>(gated(to_float<OutT>(gsrc[e]), to_float<OutT>(usrc[e]), act));
            *reinterpret_cast<uint4*>(out + (size_t)rr * ldo + n0 + seg * 8) = *reinterpret_cast<const uint4*>(res);
          }
        } else {
          const int seg = ep_tid & 15;  // 16 segments of 8 features
          const int nn = nt * BM + seg * 8;
          const bool vec_ok = ((N & 7) == 0) && ((ldo & 7) == 0);
          uint32_t epoch = 0;
          if (cm.on) epoch = *cm.epoch_word + 1u;
          for (int rr = ep_tid >> 4; rr < BN; rr += 8) {
            if (rr >= T) break;
            const OutT* src = tile + rr * kTileStride + seg * 8;
            OutT* dst = out + (size_t)rr * ldo + nn;
            if (vec_ok && nn + 8 <= N) {
              const uint4 v = *reinterpret_cast<const uint4*>(src);
              *reinterpret_cast<uint4*>(dst) = v;
              if (cm.on) {
                // {2 x 16-bit, epoch} units into slot [parity][my rank] of every peer
                const int parity = epoch & 1;
                const int64_t off = ((int64_t)parity * cm.nranks + cm.rank) * cm.slot_bytes + (int64_t)rr * N * 4 +
                                    (int64_t)nn * 4;
                for (int d = 0; d < cm.nranks; ++d) {
                  if (d == cm.rank) continue;
                  uint8_t* p = reinterpret_cast<uint8_t*>(cm.ll_bufs[d]) + off;
                  st_volatile_v4(p, v.x, epoch, v.y, epoch);
                  st_volatile_v4(p + 16, v.z, epoch, v.w, epoch);
                }
              }
            } else {
              for (int e = 0; e < 8; ++e)
                if (nn + e < N) dst[e] = src[e];
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (S > 1) {  // no CTA leaves while a peer may still write into (or read) cluster shared memory
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kCols);
  }
}

template <int BN, typename OutT, bool kFp8>
static cudaError_t launch(const GemmDecodeArgs& a, const CUtensorMap& tmW, const CUtensorMap& tmX, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_decode_kernel<BN, OutT, kFp8>;
  const int fixed = 1024 /*align*/ + 512 /*barriers*/ + (a.S - 1) * C::kSlotBytes + C::kTileBytes + 64;
  const int stage_bytes = a.w4 ? BN * BK * 2 + kPackedBytes : C::kStageBytes;
  const int a_ring = a.w4 ? kW4Tiles * kStageBytesA : 0;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, 220 * 1024);
    if (e != cudaSuccess) return e;
  }
  const int total_kb = (a.K + ((kFp8 || a.i8) ? 128 : BK) - 1) / ((kFp8 || a.i8) ? 128 : BK);
  const int nkb = a.kb_per_cta;
  // shared memory per CTA: about half an SM when two CTAs should be resident together
  int budget = (a.ctas_per_sm >= 2 ? 112 * 1024 : 216 * 1024) - fixed - a_ring;
  int stages = a.stages > 0 ? a.stages : budget / stage_bytes;
  if (stages > nkb) stages = nkb;
  if (stages > (a.w4 ? 16 : 12)) stages = a.w4 ? 16 : 12;
  if (stages < 2) stages = 2;
  const size_t smem = (size_t)stages * stage_bytes + fixed + a_ring;
  (void)total_kb;
  Comm cm;
  for (int i = 0; i < 8; ++i) cm.ll_bufs[i] = a.ll_bufs[i];
  cm.epoch_word = (const uint32_t*)a.epoch_word;
  cm.slot_bytes = a.ll_slot_bytes; cm.on = a.ar_on; cm.rank = a.rank; cm.nranks = a.nranks;
  QkvEpi qk;
  qk.positions = a.qk_positions; qk.cos_sin = a.qk_cos_sin; qk.q_w = a.qk_q_w; qk.k_w = a.qk_k_w;
  qk.kv_cache = a.qk_kv_cache; qk.slots = a.qk_slots; qk.num_blocks = a.qk_num_blocks; qk.max_pos = a.qk_max_pos;
  qk.eps = a.qk_eps; qk.on = a.qk_on; qk.Hq = a.qk_hq; qk.Hkv = a.qk_hkv; qk.neox = a.qk_neox; qk.gemma = a.qk_gemma;
  qk.block_size = a.qk_block_size;
  W4 w4p;
  w4p.scale = a.w4_scale; w4p.zero = a.w4_zero; w4p.group = a.w4_group; w4p.on = a.w4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.n_tiles * a.S);
  cfg.blockDim = dim3(a.w4 ? kThreadsW4 : kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = a.S;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, (OutT*)a.out, (const OutT*)a.bias, a.status, a.T, a.N, a.K,
                            a.kb_per_cta, a.i8 ? 2 : a.fmt, a.ldo, stages, a.S, a.act, gemm_l2_prefetch(), a.a_scale, a.w_scale,
                            a.a_stride, cm, qk, w4p);
}

}  // namespace dec
}  // namespace b200

extern "C" int b200_gemm_decode_launch(const GemmDecodeArgs* a, const void* tmW, const void* tmX, cudaStream_t st) {
  using namespace b200;
  const CUtensorMap& w = *reinterpret_cast<const CUtensorMap*>(tmW);
  const CUtensorMap& x = *reinterpret_cast<const CUtensorMap*>(tmX);
  if (a->S < 1 || a->S > 8 || a->T > a->bn || a->kb_per_cta < 1) return (int)cudaErrorInvalidValue;
  const int bke = (a->fp8 || a->i8) ? 128 : 64;
  if ((a->S - 1) * a->kb_per_cta >= (a->K + bke - 1) / bke && a->S > 1) return (int)cudaErrorInvalidValue;  // an empty CTA
  if (a->bn == 32 && a->S > 4) return (int)cudaErrorInvalidValue;
  if (a->fp8 && (a->act != 0 || a->a_scale == nullptr || a->w_scale == nullptr)) return (int)cudaErrorInvalidValue;
  if (a->i8 && (a->fp8 || a->act != 0 || a->ar_on || a->qk_on || a->a_scale == nullptr || a->w_scale == nullptr))
    return (int)cudaErrorInvalidValue;
  if (a->w4 && (a->fp8 || a->i8 || a->K % 64 != 0 || a->w4_group < 64 || a->w4_group % 64 != 0 || a->K % a->w4_group != 0 ||
                a->w4_scale == nullptr || a->w4_zero == nullptr))
    return (int)cudaErrorInvalidValue;
  if (a->qk_on && (a->fp8 || a->act != 0 || a->ar_on || a->N != (a->qk_hq + 2 * a->qk_hkv) * 128 ||
                   a->qk_positions == nullptr || a->qk_cos_sin == nullptr))
    return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaErrorInvalidValue;
  // fmt gives the OUTPUT type for fp8 inputs (1 = bf16, 0 = fp16)
  if (a->fp8) {
    if (a->bn == 16) e = (a->fmt == 1) ? dec::launch<16, __nv_bfloat16, true>(*a, w, x, st) : dec::launch<16, __half, true>(*a, w, x, st);
    else if (a->bn == 32) e = (a->fmt == 1) ? dec::launch<32, __nv_bfloat16, true>(*a, w, x, st) : dec::launch<32, __half, true>(*a, w, x, st);
  } else {
    if (a->bn == 16) e = (a->fmt == 1) ? dec::launch<16, __nv_bfloat16, false>(*a, w, x, st) : dec::launch<16, __half, false>(*a, w, x, st);
    else if (a->bn == 32) e = (a->fmt == 1) ? dec::launch<32, __nv_bfloat16, false>(*a, w, x, st) : dec::launch<32, __half, false>(*a, w, x, st);
  }
  return (int)e;
}
