// Grouped and/or fp8 block-scaled GEMM for sm_100a (tcgen05 + TMEM + TMA):
//
//   out[r, n] = sum_k x[r, k] * W[e(r), n, k]        rows r sorted by expert, lod[e] .. lod[e+1]
//
// * bf16 / fp16 inputs, or fp8 e4m3 inputs with 128x128 weight block scales (W ~ Wq * ws[e][n/128][k/128])
//   and 1x128 activation scales (x ~ xq * as[k/128][r], stored transposed).
// * lod == nullptr: one group with all T rows (a plain dense GEMM; the fp8 linear layers use this).
//
// Same orientation as gemm_bf16.cu: 128 weight rows are the UMMA M side (one per TMEM lane), BN
// token rows the N side.  Tiles never straddle experts: a token tile that runs past lod[e+1]
// computes the next expert's rows against the wrong weights and the epilogue masks them.
//
// fp8: every k-block of 128 is accumulated by the tensor core into its own TMEM buffer (two
// buffers ping-pong per k-block); the epilogue warps load it, multiply column t by
// as[kb][t] * ws[e][nt][kb] and add into fp32 registers - the scale "promotion" happens in
// software between k-blocks, overlapped with the next k-block's MMAs.
//
// The tile list depends on lod (device data), so the grid is persistent (one CTA per SM) and every
// role walks the same list: a prefix of tile counts per expert lives in shared memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "gemm_common.cuh"

namespace b200 {

constexpr int GBM = 128;
constexpr int kGThreads = 192;
constexpr int kGMaxExperts = 512;

template <int BN, bool kFp8>
struct GCfg {
  static constexpr int kElem = kFp8 ? 1 : 2;
  static constexpr int BK = 128 / kElem;                 // one 128-byte swizzle row
  static constexpr int UK = 32 / kElem;                  // K per tcgen05.mma
  static constexpr int kStageBytesA = GBM * 128;
  static constexpr int kStageBytesB = BN * 128;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  // accumulator buffers in TMEM: the fp8 path hands one over per k-block, so a deeper ring hides the hand-off
  // latency (commit -> barrier -> tcgen05.ld -> arrive); 4 x BN columns fit for BN <= 128
  static constexpr int kAccBufs = (kFp8 && BN <= 128) ? 4 : 2;
  static constexpr int kTmemCols = (kAccBufs * BN < 32) ? 32 : kAccBufs * BN;
};

struct GParams {
  void* out;            // [M, ldo]
  const void* bias;     // [E, N] or null (OutT)
  const int* lod;       // [E + 1] or null
  const float* a_scale; // fp8: [K/128, a_stride] (transposed activation scales)
  const float* w_scale; // fp8: [E, ceil(N/128), ceil(K/128)]
  int* status;
  int M, N, K, E, ldo, a_stride, fmt, num_stages, bn_rows_per_expert_hint;
};

template <int BN, bool kFp8, typename OutT>
__global__ void __launch_bounds__(kGThreads)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GParams p) {
  using Cfg = GCfg<BN, kFp8>;
  constexpr int BK = Cfg::BK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int num_stages = p.num_stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + num_stages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + num_stages;
  constexpr int NB = Cfg::kAccBufs;
  uint64_t* tmem_full = bars + 2 * num_stages;  // [NB]
  uint64_t* tmem_empty = tmem_full + NB;        // [NB]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  volatile int* ep_ok_slot = reinterpret_cast<volatile int*>(tmem_base_slot + 2);  // [2]
  int* tile_start = reinterpret_cast<int*>(tmem_base_slot + 4);                     // [E + 1]
  // [4 warps][2][BN] (fp8), read with 16-byte vector loads -> round the address up to 16 bytes
  float* sc_smem = reinterpret_cast<float*>(
      (reinterpret_cast<uintptr_t>(tile_start + kGMaxExperts + 1) + 15) & ~uintptr_t(15));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (p.K + BK - 1) / BK;
  const int n_tiles = (p.N + GBM - 1) / GBM;
  const int E = p.lod ? p.E : 1;
  Abort ab{p.status, abort_flag};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < num_stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < NB; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    mbar_fence_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
    griddep_launch();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  // lod is produced by the previous kernel (routing / permutation)
  griddep_wait();
  if (warp == 2) {
    // exclusive prefix of tiles per expert (E <= 512): lane-strided scan
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      int e = e0 + lane;
      int cnt = 0;
      if (e < E) {
        int rows = p.lod ? (p.lod[e + 1] - p.lod[e]) : p.M;
        cnt = ((rows + BN - 1) / BN) * n_tiles;
      }
      int inc = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffff, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) tile_start[e] = run + inc - cnt;
      run += __shfl_sync(0xffffffff, inc, 31);
    }
    if (lane == 0) tile_start[E] = run;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = tile_start[E];

  // tile -> (expert, n_tile, row0, rows_end); experts are walked monotonically per role
  struct Cursor { int e; };
  auto locate = [&](int tile, Cursor& c, int& e, int& nt, int& row0, int& row_end) {
    while (tile >= tile_start[c.e + 1]) ++c.e;
    e = c.e;
    int local = tile - tile_start[e];
    int base = p.lod ? p.lod[e] : 0;
    int rows = p.lod ? (p.lod[e + 1] - base) : p.M;
    int mt = (rows + BN - 1) / BN;
    nt = local / mt;
    int tt = local - nt * mt;
    row0 = base + tt * BN;
    row_end = base + rows;
  };

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Cursor cur{0};
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, nt, row0, row_end;
        locate(tile, cur, e, nt, row0, row_end);
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1, ab, 111)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageBytesA;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d_hint(sa, &tmW, &full_bar[stage], kb * BK, e * p.N + nt * GBM, pol_w);
          tma_load_2d(sb, &tmX, &full_bar[stage], kb * BK, row0);
          if (++stage == num_stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < num_stages; ++s)
          for (uint32_t q = 0; q < (1u << 14); ++q)
            if (mbar_try_wait(&full_bar[s], phase) || mbar_try_wait(&full_bar[s], phase ^ 1)) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = kFp8 ? umma_idesc(GBM, BN, 0, 0) : umma_idesc(GBM, BN, p.fmt, p.fmt);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_it = 0;  // accumulator hand-offs so far (per tile for 16-bit, per k-block for fp8)
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < total_kb; ++kb) {
          const bool new_acc = kFp8 || kb == 0;
          const int buf = acc_it % NB;
          if (new_acc) {
            if (!wait_or_abort(&tmem_empty[buf], ((acc_it / NB) & 1) ^ 1, ab, 112)) { ok = false; break; }
            tc_fence_after_sync();
          }
          if (!wait_or_abort(&full_bar[stage], phase, ab, 113)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kStageBytesA;
#pragma unroll
          for (int k = 0; k < BK / Cfg::UK; ++k) {
            uint64_t da = umma_desc_k_sw128(sa + k * 32);
            uint64_t db = umma_desc_k_sw128(sb + k * 32);
            uint32_t accumulate = (kFp8 ? (k > 0) : (kb > 0 || k > 0)) ? 1u : 0u;
            if (kFp8) umma_f8(d_tmem, da, db, idesc, accumulate);
            else umma_f16(d_tmem, da, db, idesc, accumulate);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == num_stages) { stage = 0; phase ^= 1; }
          if (kFp8 || kb == total_kb - 1) {
            umma_commit(&tmem_full[buf]);
            ++acc_it;
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int ep_tid = (warp - 2) * 32 + lane;
    float* my_sc = sc_smem + (warp - 2) * 2 * BN;
    uint32_t acc_it = 0;
    bool ok = true;
    Cursor cur{0};
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int e, nt, row0, row_end;
      locate(tile, cur, e, nt, row0, row_end);
      const int n = nt * GBM + quarter * 32 + lane;
      const bool n_ok = n < p.N;
      const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16);
      float acc[kFp8 ? BN : 1];
      if (kFp8) {
#pragma unroll
        for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      }
      const int kb_rounds = kFp8 ? total_kb : 1;
      // The scales of a k-block are fetched one k-block ahead into registers: a dependent global load in front of
      // every TMEM hand-off would otherwise bound the kernel at one L2 round trip per 16 KB of weights.
      constexpr int kScPerLane = (BN + 31) / 32;
      const int nkb = (p.K + 127) / 128;
      float a_next[kScPerLane];
      float w_next = 0.f;
      auto fetch_scales = [&](int kb) {
        w_next = p.w_scale[((size_t)e * n_tiles + nt) * nkb + kb];
#pragma unroll
        for (int i = 0; i < kScPerLane; ++i) {
          const int j = lane + 32 * i, r = row0 + j;
          a_next[i] = (j < BN && r < row_end) ? p.a_scale[(size_t)kb * p.a_stride + r] : 0.f;
        }
      };
      if (kFp8) fetch_scales(0);
      for (int kb = 0; kb < kb_rounds && ok; ++kb, ++acc_it) {
        const int buf = acc_it % NB;
        const uint32_t ph = (acc_it / NB) & 1;
        if (kFp8) {
          // stage this k-block's column scales (activation scale x weight block scale) per warp
          float* dst = my_sc + (kb & 1) * BN;
#pragma unroll
          for (int i = 0; i < kScPerLane; ++i) {
            const int j = lane + 32 * i;
            if (j < BN) dst[j] = a_next[i] * w_next;
          }
          __syncwarp();
          if (kb + 1 < kb_rounds) fetch_scales(kb + 1);
        }
        if (ep_tid == 0) ep_ok_slot[acc_it & 1] = wait_or_abort(&tmem_full[buf], ph, ab, 114) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_ok_slot[acc_it & 1] == 0) { ok = false; break; }
        while (!mbar_try_wait(&tmem_full[buf], ph)) {}
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + buf * BN + lane_addr;
        if (kFp8) {
          const float* sc = my_sc + (kb & 1) * BN;
#pragma unroll
          for (int c = 0; c < BN; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(taddr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              float4 s4 = *reinterpret_cast<const float4*>(sc + c + j);
              acc[c + j + 0] = fmaf(__uint_as_float(r[j + 0]), s4.x, acc[c + j + 0]);
              acc[c + j + 1] = fmaf(__uint_as_float(r[j + 1]), s4.y, acc[c + j + 1]);
              acc[c + j + 2] = fmaf(__uint_as_float(r[j + 2]), s4.z, acc[c + j + 2]);
              acc[c + j + 3] = fmaf(__uint_as_float(r[j + 3]), s4.w, acc[c + j + 3]);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        } else {
          float bv = (p.bias != nullptr && n_ok) ? to_float<OutT>(reinterpret_cast<const OutT*>(p.bias)[(size_t)e * p.N + n]) : 0.f;
#pragma unroll
          for (int c = 0; c < BN; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(taddr + c, r);
            tmem_ld_wait();
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                int row = row0 + c + j;
                if (row < row_end)
                  reinterpret_cast<OutT*>(p.out)[(size_t)row * p.ldo + n] = from_float<OutT>(__uint_as_float(r[j]) + bv);
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
      }
      if (kFp8 && ok && n_ok) {
        float bv = (p.bias != nullptr) ? to_float<OutT>(reinterpret_cast<const OutT*>(p.bias)[(size_t)e * p.N + n]) : 0.f;
#pragma unroll
        for (int j = 0; j < BN; ++j) {
          int row = row0 + j;
          if (row < row_end) reinterpret_cast<OutT*>(p.out)[(size_t)row * p.ldo + n] = from_float<OutT>(acc[j] + bv);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool kFp8, typename OutT>
static cudaError_t launch_grouped(const GroupedGemmArgs& a, const CUtensorMap& tmW, const CUtensorMap& tmX,
                                  cudaStream_t st) {
  using Cfg = GCfg<BN, kFp8>;
  auto kern = gemm_grouped_kernel<BN, kFp8, OutT>;
  const int extra = 1024 /*align*/ + 512 /*barriers*/ + (kGMaxExperts + 1) * 4 + 4 * 2 * BN * 4 + 64;
  int budget = 200 * 1024;
  if (BN <= 64) budget = 110 * 1024;  // leave room for the next kernel's CTA (PDL)
  int stages = (budget - extra) / Cfg::kStageBytes;
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  int smem = stages * Cfg::kStageBytes + extra;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, smem);
    if (e != cudaSuccess) return e;
  }
  GParams p;
  p.out = a.out; p.bias = a.bias; p.lod = a.lod; p.a_scale = a.a_scale; p.w_scale = a.w_scale; p.status = a.status;
  p.M = a.M; p.N = a.N; p.K = a.K; p.E = a.E; p.ldo = a.ldo; p.a_stride = a.a_stride; p.fmt = a.fmt;
  p.num_stages = stages; p.bn_rows_per_expert_hint = 0;
  return launch_pdl(kern, dim3(a.grid), dim3(kGThreads), (size_t)smem, st, tmW, tmX, p);
}

}  // namespace b200

extern "C" int b200_grouped_gemm_launch(const GroupedGemmArgs* a, const void* tmW, const void* tmX, cudaStream_t st) {
  using namespace b200;
  if (a->E > kGMaxExperts) return 2;
  const CUtensorMap& w = *reinterpret_cast<const CUtensorMap*>(tmW);
  const CUtensorMap& x = *reinterpret_cast<const CUtensorMap*>(tmX);
  cudaError_t e = cudaErrorInvalidValue;
#define B200_G_CASE(BN_)                                                                                     \
  case BN_:                                                                                                  \
    if (a->fp8) e = (a->out_fmt == 1) ? launch_grouped<BN_, true, __nv_bfloat16>(*a, w, x, st)               \
                                      : launch_grouped<BN_, true, __half>(*a, w, x, st);                     \
    else e = (a->fmt == 1) ? launch_grouped<BN_, false, __nv_bfloat16>(*a, w, x, st)                         \
                           : launch_grouped<BN_, false, __half>(*a, w, x, st);                               \
    break;
  switch (a->bn) {
    B200_G_CASE(16)
    B200_G_CASE(32)
    B200_G_CASE(64)
    B200_G_CASE(128)
    default: break;
  }
#undef B200_G_CASE
  return (int)e;
}
