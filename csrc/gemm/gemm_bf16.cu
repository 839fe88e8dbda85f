// bf16/fp16 GEMM for sm_100a:  out[T, N] = x[T, K] . W[N, K]^T (+ bias[N]),  fp32 accumulation.
//
// Orientation: the weight rows are the UMMA "M" side (128 output features per tile, one per TMEM
// lane) and the tokens are the UMMA "N" side (BN = 16..256 columns).  A decode batch of 16 tokens
// therefore wastes no tensor-core rows and the kernel streams the weight matrix once at HBM rate;
// a prefill chunk uses BN = 256.  The same kernel serves both.
//
// Structure (192 threads, persistent over work items):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tiles (128B swizzle) into a ring of stages
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected thread), commits to mbarriers
//   warps 2-5   epilogue: tcgen05.ld the accumulator (double-buffered in TMEM so the next tile's
//               main loop overlaps), add bias, convert, store; or write split-K partials
// Split-K: partial tiles go to an fp32 workspace; the last CTA to arrive for a tile (atomic ticket)
// sums the partials in a fixed order and writes the output, so results are deterministic.
// Every mbarrier wait is bounded; on time-out the CTA records a code in `status`, drains its
// outstanding copies, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "gemm_common.cuh"

namespace b200 {

constexpr int BM = 128;      // features per tile (TMEM lanes)
constexpr int BK = 64;       // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int UMMA_K = 16;   // K per tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;
constexpr int kSmemBudget = 200 * 1024;

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
};

// Collective fusion over NVLink peer memory (all pointers are peer mappings in this process):
//  * reduce-scatter epilogue: token t belongs to rank t / rs_tloc; the partial output tile is stored
//    straight into that rank's staging area [src rank][local token][N] and a per-(src, token tile)
//    counter on the owner is bumped once per finished tile, so the transfer overlaps the math;
//  * all-gather prologue: the activation rows of a token tile were pushed into THIS rank's memory by
//    their owners; the TMA producer waits (bounded) until the tile's arrival counter is complete
//    and only then issues the (local) TMA loads of that tile.
struct GemmComm {
  void* rs_stage[8];
  uint32_t* rs_flags[8];
  const uint32_t* ag_flags;
  int rs_on, rs_tloc, rs_rank;
  int ag_on, ag_expect;
  uint32_t spin_limit;
};

constexpr int kEpChunk = 64;             // token columns staged per pass of the coalescing epilogue
constexpr int kEpStride = BM + 8;        // padded row of the staging tile (elements)

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Gated activations fused into the epilogue of a gate/up projection whose weight rows are interleaved per tile as
// [64 gate rows | 64 up rows]: act = 1 SiLU, 2 GELU (tanh), 3 clamped SwiGLU of GPT-OSS.
__device__ __forceinline__ float gated_act(float g, float u, int act) {
  if (act == 1) return g / (1.f + __expf(-g)) * u;
  if (act == 2) {
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * g * (1.f + t) * u;
  }
  g = fminf(g, 7.f);
  u = fminf(fmaxf(u, -7.f), 7.f);
  return g / (1.f + __expf(-1.702f * g)) * (u + 1.f);
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
               OutT* __restrict__ out, const OutT* __restrict__ bias, float* __restrict__ ws,
               int* __restrict__ counters, int* __restrict__ status, int T, int N, int K, int n_tiles,
               int t_tiles, int per_cta, int max_contrib, int fmt, int ldo, int num_stages, int l2_prefetch, int act,
               const float* __restrict__ a_scale, const float* __restrict__ w_scale,
               const __grid_constant__ GemmComm cm) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + num_stages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + num_stages;         // [kStages]
  uint64_t* tmem_full = bars + 2 * num_stages;     // [2]
  uint64_t* tmem_empty = tmem_full + 2;            // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* ticket_slot = reinterpret_cast<int*>(tmem_base_slot + 2);
  volatile int* ep_ok_slot = reinterpret_cast<volatile int*>(tmem_base_slot + 3);  // [2]
  OutT* smem_ep = reinterpret_cast<OutT*>((reinterpret_cast<uintptr_t>(tmem_base_slot + 6) + 15) & ~uintptr_t(15));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // fmt == 2: signed 8-bit operands on kind::i8 (whole tiles only; the host never splits K for them): a k-block is
  // then 128 K-elements (still one 128-byte swizzle row), accumulators are s32, and the epilogue multiplies by the
  // per-token activation scale a_scale [T] and the per-channel weight scale w_scale [N]
  const bool i8 = fmt == 2;
  const int bke = i8 ? 128 : BK;
  const int total_kb = (K + bke - 1) / bke;
  const int num_tiles = n_tiles * t_tiles;
  Abort ab{status, abort_flag};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
    griddep_launch();  // the next kernel may become resident and run its own prologue
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  // Work decomposition.  per_cta == 0: whole tiles, CTA b takes tiles b, b + grid, ... (prefill:
  // many tiles per SM).  per_cta > 0 ("stream-K"): the k-blocks of all tiles form one sequence of
  // num_tiles * total_kb units and CTA b owns units [b * per_cta, (b + 1) * per_cta), so every SM
  // streams the same number of weight bytes whatever the tile count; a tile cut by a CTA boundary
  // is finished through the fp32 workspace by the last CTA to arrive.
  struct Work {
    int cur, end, stride, total_kb, num_tiles;
    bool streamk;
    __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1) {
      if (!streamk) {
        if (cur >= num_tiles) return false;
        tile = cur; kb0 = 0; kb1 = total_kb; cur += stride;
        return true;
      }
      if (cur >= end) return false;
      tile = cur / total_kb;
      kb0 = cur - tile * total_kb;
      int len = min(total_kb - kb0, end - cur);
      kb1 = kb0 + len;
      cur += len;
      return true;
    }
  };
  auto make_work = [&]() {
    Work w;
    w.total_kb = total_kb; w.num_tiles = num_tiles; w.streamk = per_cta > 0;
    if (per_cta > 0) {
      w.cur = blockIdx.x * per_cta;
      w.end = min(num_tiles * total_kb, w.cur + per_cta);
      w.stride = 0;
    } else {
      w.cur = blockIdx.x; w.end = 0; w.stride = gridDim.x;
    }
    return w;
  };
  // tile -> (n_tile, t_tile): groups of 8 token tiles sweep the feature tiles so that concurrently
  // resident CTAs share x and W tiles in L2.
  auto tile_coords = [&](int tile, int& nt, int& tt) {
    constexpr int G = 8;
    int group_sz = G * n_tiles;
    int g = tile / group_sz;
    int rem = tile - g * group_sz;
    int g_rows = min(G, t_tiles - g * G);
    nt = rem / g_rows;
    tt = g * G + rem % g_rows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const uint64_t pol_w = (t_tiles <= 2) ? policy_evict_first() : policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      // Weights do not depend on the previous kernel: stream the first num_stages weight tiles
      // before waiting for it, so HBM stays busy across the kernel boundary.  The activation tile
      // of each of those stages is added after the wait (one barrier, two copies).
      // For decode-shaped calls (weights are read once, the kernel is bandwidth bound) the weight tiles that
      // follow the ring are pulled into L2 as well: the kernel in front of a GEMM is usually a short
      // normalisation / activation / merge kernel that leaves HBM idle, and this CTA is already resident beside it.
      int pre = 0;
      {
        int l2_ahead = (t_tiles <= 2) ? l2_prefetch : 0;
        Work w2 = make_work();
        int tile, kb0, kb1;
        while ((pre < num_stages || l2_ahead > 0) && w2.next(tile, kb0, kb1)) {
          int nt, tt;
          tile_coords(tile, nt, tt);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (pre < num_stages) {
              mbar_expect_tx(&full_bar[pre], Cfg::kStageBytes);
              tma_load_2d_hint(smem + pre * Cfg::kStageBytes, &tmW, &full_bar[pre], kb * bke, nt * BM, pol_w);
              ++pre;
            } else if (l2_ahead > 0) {
              tma_prefetch_l2_2d(&tmW, kb * bke, nt * BM);
              --l2_ahead;
            } else {
              break;
            }
          }
        }
      }
      griddep_wait();
      Work work = make_work();
      int tile, kb0, kb1;
      while (ok && work.next(tile, kb0, kb1)) {
        int nt, tt;
        tile_coords(tile, nt, tt);
        if (cm.ag_on) {
          // rows of this token tile are pushed by their owner ranks; wait until all have landed
          bool arrived = false;
          for (uint32_t i = 0; i < cm.spin_limit; ++i) {
            if (ld_acquire_sys_u32(cm.ag_flags + tt) >= (uint32_t)cm.ag_expect) { arrived = true; break; }
            if (i > 32) __nanosleep(40);
            if ((i & 1023) == 1023 && ab.aborted()) break;
          }
          if (!arrived) { ab.raise(105); ok = false; break; }
          fence_proxy_async_global();  // peer (generic-proxy) stores -> this CTA's TMA reads
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageBytesA;
          if (issued < pre) {
            tma_load_2d(sb, &tmX, &full_bar[stage], kb * bke, tt * BN);
          } else {
            if (!wait_or_abort(&empty_bar[stage], phase ^ 1, ab, 101)) { ok = false; break; }
            mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            tma_load_2d_hint(sa, &tmW, &full_bar[stage], kb * bke, nt * BM, pol_w);
            tma_load_2d(sb, &tmX, &full_bar[stage], kb * bke, tt * BN);
          }
          ++issued;
          if (++stage == num_stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Drain: copies already issued must land before this CTA's shared memory is released.
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
      // The first full barrier completes only after the producer's own dependency wait (the activations come from
      // the previous kernel).  Waiting for the dependency here, unbounded by nature, keeps the bounded wait below
      // for what it is meant for - the copies - however long the previous kernel (say, an all-reduce that waits
      // for a late peer) takes.
      griddep_wait();
      const uint32_t idesc = i8 ? umma_idesc_i8(BM, BN) : umma_idesc(BM, BN, fmt, fmt);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      Work work = make_work();
      int tile, kb0, kb1;
      for (; ok && work.next(tile, kb0, kb1); ++local) {
        int buf = local & 1;
        uint32_t acc_phase = (local >> 1) & 1;
        if (!wait_or_abort(&tmem_empty[buf], acc_phase ^ 1, ab, 102)) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full_bar[stage], phase, ab, 103)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          uint32_t sb = sa + Cfg::kStageBytesA;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = umma_desc_k_sw128(sa + k * UMMA_K * 2);
            uint64_t db = umma_desc_k_sw128(sb + k * UMMA_K * 2);
            if (i8) umma_i8(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_f16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == num_stages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    const int ep_tid = (warp - 2) * 32 + lane;
    int local = 0;
    bool ok = true;
    griddep_wait();  // before the first global write / workspace access of this CTA
    Work work = make_work();
    int tile, kb0, kb1;
    for (; ok && work.next(tile, kb0, kb1); ++local) {
      int nt, tt;
      tile_coords(tile, nt, tt);
      int buf = local & 1;
      uint32_t acc_phase = (local >> 1) & 1;
      // One thread does the bounded wait and publishes the outcome, so that the 128 epilogue
      // threads always agree and none is left alone at a named barrier.
      // (two flag slots: thread 0 may already be publishing for the next item while a slow thread reads)
      if (ep_tid == 0) ep_ok_slot[local & 1] = wait_or_abort(&tmem_full[buf], acc_phase, ab, 104) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ep_ok_slot[local & 1] == 0) { ok = false; break; }
      while (!mbar_try_wait(&tmem_full[buf], acc_phase)) {}  // phase is complete: returns at once
      tc_fence_after_sync();
      const int n = nt * BM + quarter * 32 + lane;
      const int t0 = tt * BN;
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      const bool n_ok = n < N;
      if (kb0 == 0 && kb1 == total_kb) {
        float bv = (bias != nullptr && n_ok) ? to_float<OutT>(bias[n]) : 0.f;
        const float wsc = (i8 && n_ok) ? w_scale[n] : 0.f;
        // accumulator word of token t -> real value (+ bias)
        auto val = [&](uint32_t r, int t) -> float {
          if (i8) return (float)(int)r * wsc * (t < T ? a_scale[t] : 0.f) + bv;
          return __uint_as_float(r) + bv;
        };
        // destination row of token t: the local output, or the owner rank's staging area
        auto row_ptr = [&](int t) -> OutT* {
          if (cm.rs_on) {
            int owner = t / cm.rs_tloc;
            int tl = t - owner * cm.rs_tloc;
            return reinterpret_cast<OutT*>(cm.rs_stage[owner]) + ((size_t)cm.rs_rank * cm.rs_tloc + tl) * N;
          }
          return out + (size_t)t * ldo;
        };
        if (act != 0) {
          // gate / up tile: stage [token][128] in shared memory (rounded to OutT, as an unfused projection would hand
          // it to the activation kernel), then every thread combines 8 gate features with their 8 up features and
          // writes 16 bytes of the half-width output row
          constexpr int kChunk = BN < kEpChunk ? BN : kEpChunk;
          const int n_local = quarter * 32 + lane;
          const int n0 = nt * (BM / 2);
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += kChunk) {
            if (t0 + c0 < T) {
#pragma unroll
              for (int c = 0; c < kChunk; c += 16) {
                uint32_t r[16];
                tmem_ld_x16(taddr + c0 + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  smem_ep[(c + j) * kEpStride + n_local] = from_float<OutT>(__uint_as_float(r[j]) + bv);
              }
            }
            if (c0 + kChunk >= BN) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (t0 + c0 < T) {
              const int seg = ep_tid & 7;            // 8 segments of 8 output features
              for (int rr = ep_tid >> 3; rr < kChunk; rr += 16) {
                const int t = t0 + c0 + rr;
                if (t >= T) break;
                const OutT* gsrc = smem_ep + rr * kEpStride + seg * 8;
                const OutT* usrc = gsrc + BM / 2;
                alignas(16) OutT res[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  res[e] = from_float<OutT>(gated_act(to_float<OutT>(gsrc[e]), to_float<OutT>(usrc[e]), act));
                *reinterpret_cast<uint4*>(out + (size_t)t * ldo + n0 + seg * 8) = *reinterpret_cast<const uint4*>(res);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        } else if (BN >= kEpChunk) {
          // TMEM -> registers -> shared [token][feature] -> 16-byte row segments (256 B per token row)
          const int n_local = quarter * 32 + lane;
          const int n0 = nt * BM;
          const bool vec_ok = ((N & 7) == 0) && (cm.rs_on || (ldo & 7) == 0);
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += kEpChunk) {
            if (t0 + c0 < T) {
#pragma unroll
              for (int c = 0; c < kEpChunk; c += 16) {
                uint32_t r[16];
                tmem_ld_x16(taddr + c0 + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  smem_ep[(c + j) * kEpStride + n_local] = from_float<OutT>(val(r[j], t0 + c0 + c + j));
              }
            }
            if (c0 + kEpChunk >= BN) {  // accumulator fully read: hand the TMEM buffer back
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (t0 + c0 < T) {
              const int seg = ep_tid & 15;           // 16 segments of 8 features
              const int nn = n0 + seg * 8;
              for (int rr = ep_tid >> 4; rr < kEpChunk; rr += 8) {
                const int t = t0 + c0 + rr;
                if (t >= T) break;
                OutT* dst = row_ptr(t) + nn;
                const OutT* src = smem_ep + rr * kEpStride + seg * 8;
                if (vec_ok && nn + 8 <= N) {
                  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                  for (int e = 0; e < 8; ++e)
                    if (nn + e < N) dst[e] = src[e];
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        } else {
#pragma unroll
          for (int c = 0; c < BN; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(taddr + c, r);
            tmem_ld_wait();
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                int t = t0 + c + j;
                if (t < T) row_ptr(t)[n] = from_float<OutT>(val(r[j], t));
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        if (cm.rs_on) {
          // tile delivered: publish it on the owner (one arrival per tile)
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (ep_tid == 0) {
            int owner = t0 / cm.rs_tloc;
            int tl0 = t0 - owner * cm.rs_tloc;
            red_release_sys_add(cm.rs_flags[owner] + tl0 / BN, 1u);
          }
        }
      } else {
        // partial tile -> workspace [tile][slot][BN][128]; slot = rank of this CTA among the CTAs
        // whose unit ranges intersect the tile (ascending K order)
        const int first_cta = (tile * total_kb) / per_cta;
        const int last_cta = ((tile + 1) * total_kb - 1) / per_cta;
        const int contrib = last_cta - first_cta + 1;
        const int slot = (int)blockIdx.x - first_cta;
        float* wtile = ws + ((size_t)tile * max_contrib + slot) * (BN * BM);
#pragma unroll
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) wtile[(c + j) * BM + quarter * 32 + lane] = __uint_as_float(r[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) {
          int prev = atomicAdd(&counters[tile], 1);
          if (prev == contrib - 1) counters[tile] = 0;  // re-arm for the next launch / graph replay
          *ticket_slot = prev;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*ticket_slot == contrib - 1) {
          __threadfence();
          const float* wbase = ws + (size_t)tile * max_contrib * (BN * BM) + quarter * 32 + lane;
          float bv = (bias != nullptr && n_ok) ? to_float<OutT>(bias[n]) : 0.f;
          // 16 columns x 2 slots per round: 32 independent loads are in flight before the first add,
          // and slots are summed in ascending K order (deterministic).
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (t0 + c0 >= T) break;
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = bv;
            int s = 0;
            for (; s + 2 <= contrib; s += 2) {
              const float* wp = wbase + (size_t)s * (BN * BM) + c0 * BM;
              float v0[16], v1[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) { v0[j] = __ldcg(wp + j * BM); v1[j] = __ldcg(wp + BN * BM + j * BM); }
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = (acc[j] + v0[j]) + v1[j];
            }
            if (s < contrib) {
              const float* wp = wbase + (size_t)s * (BN * BM) + c0 * BM;
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] += __ldcg(wp + j * BM);
            }
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                int t = t0 + c0 + j;
                if (t < T) out[(size_t)t * ldo + n] = from_float<OutT>(acc[j]);
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // ticket_slot is reused by the next item
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

template <int BN, typename OutT>
static cudaError_t launch_bn(const GemmArgs& a, const CUtensorMap& tmW, const CUtensorMap& tmX, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tn_kernel<BN, OutT>;
  constexpr int kEpBytes = (BN >= kEpChunk ? kEpChunk : BN) * kEpStride * 2 + 64;  // staging tile of the epilogue
  GemmComm cm;
  for (int i = 0; i < 8; ++i) { cm.rs_stage[i] = a.rs_stage[i]; cm.rs_flags[i] = (uint32_t*)a.rs_flags[i]; }
  cm.ag_flags = (const uint32_t*)a.ag_flags;
  cm.rs_on = a.rs_on; cm.rs_tloc = a.rs_tloc; cm.rs_rank = a.rs_rank; cm.ag_on = a.ag_on; cm.ag_expect = a.ag_expect;
  cm.spin_limit = a.spin_limit;
  {
    cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kStagesRaw * Cfg::kStageBytes + 1024 + 512 + kEpBytes);
    if (e != cudaSuccess) return e;
  }
  // Shared memory per CTA decides how many CTAs share an SM: small token tiles run two CTAs per SM
  // so one CTA's prologue / split-K epilogue overlaps the other's main loop.
  int ctas_per_sm = a.ctas_per_sm > 0 ? a.ctas_per_sm : 1;
  int budget = (kSmemBudget + 24 * 1024) / ctas_per_sm - 2048 - kEpBytes;
  int stages = a.stages > 0 ? a.stages : budget / Cfg::kStageBytes;
  // decode-sized token tiles: keep a CTA near 110 KB so the next GEMM's CTA can become resident
  // beside it (PDL) and start prefetching its weights while this one drains
  if (a.stages <= 0 && BN <= 64 && a.t_tiles == 1 && stages > 6) stages = 6;
  if (stages > 12) stages = 12;
  if (stages > Cfg::kStagesRaw) stages = Cfg::kStagesRaw;
  if (stages < 2) stages = 2;
  int smem = stages * Cfg::kStageBytes + 1024 + 512 + kEpBytes;
  return launch_pdl(kern, dim3(a.grid), dim3(kGemmThreads), (size_t)smem, st, tmW, tmX, (OutT*)a.out,
                    (const OutT*)a.bias, a.ws, a.counters, a.status, a.T, a.N, a.K, a.n_tiles, a.t_tiles, a.per_cta,
                    a.max_contrib, a.i8 ? 2 : a.fmt, a.ldo, stages, b200::gemm_l2_prefetch(), a.act, a.a_scale, a.w_scale,
                    cm);
}

}  // namespace b200

extern "C" int b200_gemm_pick_bn(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  if (T <= 256) return 256;
  int pad128 = (T + 127) / 128 * 128, pad256 = (T + 255) / 256 * 256;
  return (pad128 < pad256) ? 128 : 256;
}

extern "C" int b200_gemm_launch(const GemmArgs* a, const void* tmW, const void* tmX, cudaStream_t st) {
  using namespace b200;
  const CUtensorMap& w = *reinterpret_cast<const CUtensorMap*>(tmW);
  const CUtensorMap& x = *reinterpret_cast<const CUtensorMap*>(tmX);
  cudaError_t e = cudaErrorInvalidValue;
  // 8-bit integer operands: whole tiles, plain epilogue, scales required
  if (a->i8 && (a->per_cta != 0 || a->act != 0 || a->rs_on || a->ag_on || a->a_scale == nullptr || a->w_scale == nullptr))
    return (int)e;
#define B200_BN_CASE(BN_)                                                                              \
  case BN_:                                                                                            \
    e = (a->fmt == 1) ? launch_bn<BN_, __nv_bfloat16>(*a, w, x, st) : launch_bn<BN_, __half>(*a, w, x, st); \
    break;
  switch (a->bn) {
    B200_BN_CASE(16)
    B200_BN_CASE(32)
    B200_BN_CASE(64)
    B200_BN_CASE(128)
    B200_BN_CASE(256)
    default: break;
  }
#undef B200_BN_CASE
  return (int)e;
}
