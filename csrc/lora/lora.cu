// Multi-adapter LoRA kernels: shrink (x @ A[id]^T * scale -> fp32 [T, r]) and expand
// (out[:, off:off+N] (+)= h @ B[id]^T), with the adapter chosen per token.  Segment-wise calls (one adapter
// per sequence, prefill) and per-token calls (decode) share the kernels: segments are expanded to a per-token
// id vector by the caller.
//
// Reference entry points: _C::sgmv_shrink_lora / sgmv_expand(_slice)_lora / bgmv_shrink_lora /
// bgmv_expand(_slice)_lora (vllm_kunlun/ops/_custom_ops.py:2435-2836), driven by PunicaWrapperKunlun
// (vllm_kunlun/lora/punica_wrapper/punica_kunlun.py:273-545).
#include <cstring>

#include "../api.h"
#include "../attention/attn_common.cuh"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/utils.cuh"

namespace b200 {
namespace {

// Shrink.  One block per tile of up to 8 consecutive tokens: the activation rows are staged in shared memory once and
// each warp walks two rank rows of A at a time, so an A vector read from L2 serves every token of the tile that uses
// that adapter and an activation vector read from shared memory serves two rank rows (one block per token re-read
// all of A from L2 for every token).  A tile makes one pass per distinct adapter among its tokens: one pass for the
// runs of a prefill segment, a few for decode batches that mix adapters.
constexpr int kShrinkTile = 8;

template <typename T>
__global__ void __launch_bounds__(256) lora_shrink_kernel(float* __restrict__ out, const T* __restrict__ x, int64_t x_stride,
                                                          const T* __restrict__ A /*[L, r, K]*/, const int* __restrict__ ids,
                                                          int64_t T_, int mt, int r, int K, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sx = reinterpret_cast<T*>(smem_raw);
  __shared__ int s_ids[kShrinkTile];
  const int64_t t0 = (int64_t)blockIdx.x * mt;
  const int n_tok = (int)min((int64_t)mt, T_ - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __shared__ __align__(8) uint64_t s_bar;
  if (threadIdx.x < kShrinkTile) s_ids[threadIdx.x] = threadIdx.x < n_tok ? ids[t0 + threadIdx.x] : -1;
  constexpr int VN = Vec16<T>::N;
  // the tile's activation rows come in as bulk copies (one per row) that complete on an mbarrier: no thread holds a
  // row in registers on the way, and the copies of the resident blocks overlap each other's arithmetic
  if (threadIdx.x == 0) {
    mbar_init(&s_bar, 1);
    mbar_fence_init();
    const uint32_t row_bytes = (uint32_t)K * sizeof(T);
    mbar_expect_tx(&s_bar, row_bytes * n_tok);
    for (int m = 0; m < n_tok; ++m) bulk_load_1d(sx + (int64_t)m * K, x + (t0 + m) * x_stride, row_bytes, &s_bar);
  }
  __syncthreads();
  if (!mbar_wait(&s_bar, 0)) {   // bounded; a copy that never lands leaves NaN, not stale numbers
    for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) out[t0 * r + j] = __int_as_float(0x7fc00000);
    return;
  }
  for (int m = 0; m < n_tok; ++m)     // base-model rows
    if (s_ids[m] < 0)
      for (int j = threadIdx.x; j < r; j += blockDim.x) out[(t0 + m) * r + j] = 0.f;
  for (int a = 0; a < n_tok; ++a) {   // one pass per distinct adapter (block-uniform control flow)
    const int d = s_ids[a];
    if (d < 0) continue;
    bool first = true;
    for (int q = 0; q < a; ++q) first = first && s_ids[q] != d;
    if (!first) continue;
    unsigned mask = 0;
    for (int m = a; m < n_tok; ++m) mask |= (s_ids[m] == d ? 1u : 0u) << m;
    for (int j = warp * 2; j < r; j += nw * 2) {
      const bool two = j + 1 < r;
      const T* a0 = A + ((int64_t)d * r + j) * K;
      const T* a1 = two ? a0 + K : a0;
      float acc0[kShrinkTile], acc1[kShrinkTile];
#pragma unroll
      for (int m = 0; m < kShrinkTile; ++m) acc0[m] = acc1[m] = 0.f;
#pragma unroll 2
      for (int i = lane * VN; i < K; i += 32 * VN) {
        Vec16<T> av0 = ld_vec(a0 + i), av1 = ld_vec(a1 + i);
        float f0[VN], f1[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) { f0[e] = to_f(av0.v[e]); f1[e] = to_f(av1.v[e]); }
#pragma unroll
        for (int m = 0; m < kShrinkTile; ++m) {
          if ((mask >> m) & 1u) {
            Vec16<T> xv = ld_vec(sx + (int64_t)m * K + i);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
              const float xe = to_f(xv.v[e]);
              acc0[m] += f0[e] * xe;
              acc1[m] += f1[e] * xe;
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < kShrinkTile; ++m) {
        if ((mask >> m) & 1u) {
          const float s0 = warp_sum(acc0[m]), s1 = warp_sum(acc1[m]);
          if (lane == 0) {
            out[(t0 + m) * r + j] = s0 * scale;
            if (two) out[(t0 + m) * r + j + 1] = s1 * scale;
          }
        }
      }
    }
  }
}

// Expand.  grid (ceil(T / 16), ceil(N / 512)): a block covers a tile of up to 16 consecutive tokens x 512 output
// columns, a thread two adjacent columns; the two B rows of a thread are read once per tile and adapter (not once per
// token) and the 16 h rows (fp32) sit in shared memory, read as broadcasts; the read-modify-write of the output is
// 4 bytes per thread, 128 contiguous bytes per warp and token.  One pass per distinct adapter of the tile.
constexpr int kExpandTile = 16;

template <typename T>
__global__ void __launch_bounds__(256) lora_expand_kernel(T* __restrict__ out, int64_t out_stride, int offset,
                                                          const float* __restrict__ h, const T* __restrict__ B /*[L, N, r]*/,
                                                          const int* __restrict__ ids, int64_t T_, int N, int r, int add,
                                                          int pair_ok) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sh = reinterpret_cast<float*>(smem_raw);      // [16][r]
  __shared__ int s_ids[kExpandTile];
  const int64_t t0 = (int64_t)blockIdx.x * kExpandTile;
  const int n_tok = (int)min((int64_t)kExpandTile, T_ - t0);
  if (threadIdx.x < kExpandTile) s_ids[threadIdx.x] = threadIdx.x < n_tok ? ids[t0 + threadIdx.x] : -1;
  for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) sh[j] = h[t0 * r + j];
  __syncthreads();
  const int n0 = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (n0 >= N) return;
  const bool two = n0 + 1 < N;
  constexpr int VN = Vec16<T>::N;
  float acc0[kExpandTile], acc1[kExpandTile];
#pragma unroll
  for (int m = 0; m < kExpandTile; ++m) acc0[m] = acc1[m] = 0.f;
  // the old output values of every adapter row are requested up front, all at once: issued one by one between the
  // stores they would be a chain of 16 memory round trips
  const bool paired = two && pair_ok && sizeof(T) == 2;
  unsigned act = 0;
  for (int m = 0; m < n_tok; ++m) act |= (s_ids[m] >= 0 ? 1u : 0u) << m;
  uint32_t old0[kExpandTile], old1[kExpandTile];
#pragma unroll
  for (int m = 0; m < kExpandTile; ++m) {
    old0[m] = old1[m] = 0u;
    if (add && ((act >> m) & 1u)) {
      const T* o = out + (t0 + m) * out_stride + offset + n0;
      if (paired) {
        old0[m] = *reinterpret_cast<const uint32_t*>(o);
      } else {
        old0[m] = __float_as_uint(to_f(o[0]));
        if (two) old1[m] = __float_as_uint(to_f(o[1]));
      }
    }
  }
  unsigned any = 0;
  for (int a = 0; a < n_tok; ++a) {   // one pass per distinct adapter
    const int d = s_ids[a];
    if (d < 0) continue;
    bool first = true;
    for (int q = 0; q < a; ++q) first = first && s_ids[q] != d;
    if (!first) continue;
    unsigned mask = 0;
    for (int m = a; m < n_tok; ++m) mask |= (s_ids[m] == d ? 1u : 0u) << m;
    any |= mask;
    const T* b0 = B + ((int64_t)d * N + n0) * r;
    const T* b1 = two ? b0 + r : b0;
    if (r % VN == 0) {
      for (int j = 0; j < r; j += VN) {
        Vec16<T> v0 = ld_vec(b0 + j), v1 = ld_vec(b1 + j);
        float f0[VN], f1[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) { f0[e] = to_f(v0.v[e]); f1[e] = to_f(v1.v[e]); }
#pragma unroll
        for (int m = 0; m < kExpandTile; ++m) {
          if ((mask >> m) & 1u) {
#pragma unroll
            for (int e = 0; e < VN; ++e) {
              const float he = sh[m * r + j + e];
              acc0[m] += f0[e] * he;
              acc1[m] += f1[e] * he;
            }
          }
        }
      }
    } else {
      for (int j = 0; j < r; ++j) {
        const float f0 = to_f(b0[j]), f1 = to_f(b1[j]);
#pragma unroll
        for (int m = 0; m < kExpandTile; ++m)
          if ((mask >> m) & 1u) { acc0[m] += f0 * sh[m * r + j]; acc1[m] += f1 * sh[m * r + j]; }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kExpandTile; ++m) {
    if ((any >> m) & 1u) {
      T* o = out + (t0 + m) * out_stride + offset + n0;
      if (paired) {   // one 4-byte access for the two columns
        uint32_t w = old0[m];
        T lo, hi;
        memcpy(&lo, &w, 2);
        memcpy(&hi, reinterpret_cast<const char*>(&w) + 2, 2);
        lo = from_f<T>(add ? to_f(lo) + acc0[m] : acc0[m]);
        hi = from_f<T>(add ? to_f(hi) + acc1[m] : acc1[m]);
        memcpy(&w, &lo, 2);
        memcpy(reinterpret_cast<char*>(&w) + 2, &hi, 2);
        *reinterpret_cast<uint32_t*>(o) = w;
      } else {
        o[0] = from_f<T>(__uint_as_float(old0[m]) + acc0[m]);
        if (two) o[1] = from_f<T>(__uint_as_float(old1[m]) + acc1[m]);
      }
    }
  }
}

// Expand through shared memory and bulk copies (aligned shapes).  Same tiling and arithmetic as above, but a thread
// never touches the output: the tile's deltas are written to shared memory in the output type and every adapter row
// of the tile then leaves as ONE bulk copy of up to 1 KB - with `add`, a bulk reduction: the memory system adds the
// row into global memory, so no thread waits for old output values and the read-modify-write never crosses the SM.
// (The delta is rounded to the output type before it is added: one extra rounding of the delta, not of the sum.)
template <typename T> __device__ __forceinline__ void bulk_reduce_add(void* dst, const void* src, uint32_t bytes);
template <> __device__ __forceinline__ void bulk_reduce_add<__nv_bfloat16>(void* dst, const void* src, uint32_t bytes) {
  bulk_reduce_add_bf16(dst, src, bytes);
}
template <> __device__ __forceinline__ void bulk_reduce_add<__half>(void* dst, const void* src, uint32_t bytes) {
  bulk_reduce_add_f16(dst, src, bytes);
}
template <> __device__ __forceinline__ void bulk_reduce_add<float>(void* dst, const void* src, uint32_t bytes) {
  bulk_reduce_add_f32(dst, src, bytes);
}

constexpr int kExpandCols = 512;

template <typename T>
__global__ void __launch_bounds__(256) lora_expand_bulk_kernel(T* __restrict__ out, int64_t out_stride, int offset,
                                                               const float* __restrict__ h, const T* __restrict__ B,
                                                               const int* __restrict__ ids, int64_t T_, int N, int r,
                                                               int add) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);                                          // [16][512] deltas
  float* sh = reinterpret_cast<float*>(smem_raw + kExpandTile * kExpandCols * sizeof(T));   // [16][r]
  __shared__ int s_ids[kExpandTile];
  const int64_t t0 = (int64_t)blockIdx.y * kExpandTile;
  const int n_tok = (int)min((int64_t)kExpandTile, T_ - t0);
  if (threadIdx.x < kExpandTile) s_ids[threadIdx.x] = threadIdx.x < n_tok ? ids[t0 + threadIdx.x] : -1;
  for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) sh[j] = h[t0 * r + j];
  __syncthreads();
  const int nb = blockIdx.x * kExpandCols;           // first column of the block
  const int n0 = nb + threadIdx.x * 2;
  constexpr int VN = Vec16<T>::N;
  if (n0 < N) {                                       // N is even here (the launcher checks alignment)
    float acc0[kExpandTile], acc1[kExpandTile];
#pragma unroll
    for (int m = 0; m < kExpandTile; ++m) acc0[m] = acc1[m] = 0.f;
    for (int a = 0; a < n_tok; ++a) {   // one pass per distinct adapter
      const int d = s_ids[a];
      if (d < 0) continue;
      bool first = true;
      for (int q = 0; q < a; ++q) first = first && s_ids[q] != d;
      if (!first) continue;
      unsigned mask = 0;
      for (int m = a; m < n_tok; ++m) mask |= (s_ids[m] == d ? 1u : 0u) << m;
      const T* b0 = B + ((int64_t)d * N + n0) * r;
      const T* b1 = b0 + r;
      for (int j = 0; j < r; j += VN) {
        Vec16<T> v0 = ld_vec(b0 + j), v1 = ld_vec(b1 + j);
        float f0[VN], f1[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) { f0[e] = to_f(v0.v[e]); f1[e] = to_f(v1.v[e]); }
#pragma unroll
        for (int m = 0; m < kExpandTile; ++m) {
          if ((mask >> m) & 1u) {
#pragma unroll
            for (int e = 0; e < VN; ++e) {
              const float he = sh[m * r + j + e];
              acc0[m] += f0[e] * he;
              acc1[m] += f1[e] * he;
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kExpandTile; ++m) {
      tile[m * kExpandCols + threadIdx.x * 2] = from_f<T>(acc0[m]);
      tile[m * kExpandCols + threadIdx.x * 2 + 1] = from_f<T>(acc1[m]);
    }
  }
  fence_proxy_async_smem();     // the deltas were written by ordinary stores; the bulk copies read them
  __syncthreads();
  if (threadIdx.x < n_tok && s_ids[threadIdx.x] >= 0) {    // one thread per adapter row: one bulk copy each
    const int m = threadIdx.x;
    const uint32_t bytes = (uint32_t)(min(kExpandCols, N - nb) * sizeof(T));
    T* dst = out + (t0 + m) * out_stride + offset + nb;
    if (add) bulk_reduce_add<T>(dst, tile + m * kExpandCols, bytes);
    else bulk_store_1d(dst, tile + m * kExpandCols, bytes);
    tma_store_commit();
    tma_store_wait_read();      // shared memory must stay until the copy has read it; the grid's end completes the writes
  }
}

// ---- 16-bit types: the two products on warp-level tensor-core MMAs (m16n8k16, fp32 accumulation).  Both are thin
// contractions (the adapter rank is the N side of shrink and the K side of expand), so they stay bound by memory once
// the arithmetic leaves the CUDA cores.  A tile whose tokens use several adapters makes one pass per adapter with the
// rows of the other tokens zeroed in the A fragments, accumulating into the same registers.

// Shrink: tile of up to 8 tokens (rows 8 - 15 of the MMA are zero), activation rows staged by bulk copies with a
// 64-byte pad per row (conflict-free 16-byte fragment loads), 32-element K chunks interleaved over the 8 warps, A
// fragments from shared memory, B fragments (adapter rows, k contiguous) straight from L2, partial sums combined
// through shared memory.  The order of the k index inside a chunk is free in a contraction, so the fragments are
// chosen to be contiguous in memory: lane (g, tq) takes elements tq * 8 .. tq * 8 + 7 of the chunk - the first four
// as its k slots of one MMA, the last four as those of a second one - for the activation row and the adapter row
// alike: one 16-byte load each per two MMAs instead of four 4-byte loads.
constexpr int kShrinkMaxRank = 64;
constexpr int kShrinkRowPad = 32;   // elements

// The tokens of a tile grouped by adapter, by the first warp: mask[m] = the tile's tokens that use the adapter of token
// m if m is the first of them, else 0 (base-model rows: 0).  One pass of the kernels below per non-zero mask.
template <int kTile>
__device__ __forceinline__ void group_by_adapter(const int* __restrict__ ids, int64_t t0, int n_tok, int* s_ids, unsigned* s_mask) {
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    const int id = lane < n_tok ? ids[t0 + lane] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, id);
    const bool first = id >= 0 && (__ffs(peers) - 1) == lane;
    if (lane < kTile) {
      s_ids[lane] = id;
      s_mask[lane] = first ? peers : 0u;
    }
  }
}

// NT = 8-wide rank tiles (r <= 8 NT); the B fragments of 8 / NT chunks are requested together before the first MMA
// of the batch, so a warp has 8 independent 16-byte loads in flight per round trip to L2.
template <typename T, int NT>
__global__ void __launch_bounds__(256) lora_shrink_mma_kernel(float* __restrict__ out, const T* __restrict__ x, int64_t x_stride,
                                                              const T* __restrict__ A /*[L, r, K]*/, const int* __restrict__ ids,
                                                              int64_t T_, int mt, int r, int K, float scale) {
  constexpr int UB = 8 / NT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int row_elems = K + kShrinkRowPad;                       // padded row
  T* sx = reinterpret_cast<T*>(smem_raw);                        // [mt][K + 32]
  float* part = reinterpret_cast<float*>(smem_raw + (size_t)mt * row_elems * sizeof(T));   // [8 warps][8][r]
  __shared__ int s_ids[kShrinkTile];
  __shared__ unsigned s_mask[kShrinkTile];
  __shared__ __align__(8) uint64_t s_bar;
  const int64_t t0 = (int64_t)blockIdx.x * mt;
  const int n_tok = (int)min((int64_t)mt, T_ - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  if (threadIdx.x == 0) {
    mbar_init(&s_bar, 1);
    mbar_fence_init();
    const uint32_t row_bytes = (uint32_t)K * sizeof(T);
    mbar_expect_tx(&s_bar, row_bytes * n_tok);
    for (int m = 0; m < n_tok; ++m) bulk_load_1d(sx + (int64_t)m * row_elems, x + (t0 + m) * x_stride, row_bytes, &s_bar);
  }
  group_by_adapter<kShrinkTile>(ids, t0, n_tok, s_ids, s_mask);
  __syncthreads();
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  const T* xrow = sx + (int64_t)g * row_elems + tq * 8;          // this lane's token row, its 8 elements of a chunk
  bool waited = false, ok = true;
  for (int a = 0; a < n_tok && ok; ++a) {   // one pass per distinct adapter
    const unsigned mask = s_mask[a];
    if (mask == 0u) continue;
    const bool mine = (mask >> g) & 1u;      // does this lane's row take part in the pass
    const T* Ad = A + (int64_t)s_ids[a] * r * K + tq * 8;
    for (int kb = warp * 32; kb < K; kb += 8 * 32 * UB) {
      uint4 b[UB][NT];
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int k0 = kb + u * 8 * 32;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int n = nt * 8 + g;
          b[u][nt] = (k0 < K && n < r) ? *reinterpret_cast<const uint4*>(Ad + (int64_t)n * K + k0) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (!waited) {   // the activation rows: bounded wait, after the first adapter loads are on their way
        ok = __all_sync(0xffffffffu, mbar_wait(&s_bar, 0));   // warp-uniform: the MMAs below are warp-collective
        waited = true;
        if (!ok) break;
      }
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int k0 = kb + u * 8 * 32;
        if (k0 < K) {
          const uint4 xa = mine ? *reinterpret_cast<const uint4*>(xrow + k0) : make_uint4(0u, 0u, 0u, 0u);
          const uint32_t af0[4] = {xa.x, 0u, xa.y, 0u}, af1[4] = {xa.z, 0u, xa.w, 0u};   // rows 8 - 15 are zero
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            MmaTraits<T>::mma(acc[nt], af0, b[u][nt].x, b[u][nt].y);
            MmaTraits<T>::mma(acc[nt], af1, b[u][nt].z, b[u][nt].w);
          }
        }
      }
    }
  }
  if (!waited) ok = mbar_wait(&s_bar, 0);    // no adapter row in the tile: the copies still own the shared memory
  // c0, c1 = (row g, columns 2 tq, 2 tq + 1) of every rank tile; rows 8 - 15 are unused
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + 2 * tq;
    if (n < r) part[(warp * 8 + g) * r + n] = acc[nt][0];
    if (n + 1 < r) part[(warp * 8 + g) * r + n + 1] = acc[nt][1];
  }
  if (__syncthreads_or(!ok)) {   // a copy that never landed leaves NaN, not stale numbers
    for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) out[t0 * r + j] = __int_as_float(0x7fc00000);
    return;
  }
  for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += part[w * 8 * r + j];
    out[t0 * r + j] = sum * scale;
  }
}

// Expand: a block covers 16 tokens x 512 columns, a warp 64 of the columns as eight 8-column MMA tiles; the A fragments
// are the tile's h rows (rounded to the 16-bit type), the B fragments the adapter's rows (rank contiguous) straight
// from L2; the deltas go to shared memory in the output type (rows padded by 16 bytes) and leave as one bulk copy /
// bulk reduction per adapter row, as in the kernel above.
constexpr int kExpandRowPad = kExpandCols + 8;

template <typename T>
__global__ void __launch_bounds__(256) lora_expand_mma_kernel(T* __restrict__ out, int64_t out_stride, int offset,
                                                              const float* __restrict__ h, const T* __restrict__ B,
                                                              const int* __restrict__ ids, int64_t T_, int N, int r,
                                                              int add) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);                                              // [16][520] deltas
  float* sh = reinterpret_cast<float*>(smem_raw + kExpandTile * kExpandRowPad * sizeof(T));   // [16][r]
  __shared__ int s_ids[kExpandTile];
  __shared__ unsigned s_mask[kExpandTile];
  const int64_t t0 = (int64_t)blockIdx.y * kExpandTile;
  const int n_tok = (int)min((int64_t)kExpandTile, T_ - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  group_by_adapter<kExpandTile>(ids, t0, n_tok, s_ids, s_mask);
  for (int j = threadIdx.x; j < n_tok * r; j += blockDim.x) sh[j] = h[t0 * r + j];
  __syncthreads();
  const int nb = blockIdx.x * kExpandCols;           // first column of the block
  const int nw = nb + warp * 64;                     // first column of the warp
  float acc[8][4];
#pragma unroll
  for (int ng = 0; ng < 8; ++ng) acc[ng][0] = acc[ng][1] = acc[ng][2] = acc[ng][3] = 0.f;
  if (nw < N) {
    for (int a = 0; a < n_tok; ++a) {   // one pass per distinct adapter
      const unsigned mask = s_mask[a];
      if (mask == 0u) continue;
      const bool lo = (mask >> g) & 1u, hi = (mask >> (g + 8)) & 1u;
      const T* Bd = B + (int64_t)s_ids[a] * N * r;
      for (int k0 = 0; k0 < r; k0 += 16) {
        // k slots of lane (g, tq): elements ka .. ka + 3 of the rank (contiguous; the order inside a k-step is free)
        const int ka = k0 + 4 * tq;
        const bool kin = ka < r;                        // r is a multiple of 4
        uint32_t af[4];
        af[0] = (lo && kin) ? MmaTraits<T>::pack(sh[g * r + ka], sh[g * r + ka + 1]) : 0u;
        af[1] = (hi && kin) ? MmaTraits<T>::pack(sh[(g + 8) * r + ka], sh[(g + 8) * r + ka + 1]) : 0u;
        af[2] = (lo && kin) ? MmaTraits<T>::pack(sh[g * r + ka + 2], sh[g * r + ka + 3]) : 0u;
        af[3] = (hi && kin) ? MmaTraits<T>::pack(sh[(g + 8) * r + ka + 2], sh[(g + 8) * r + ka + 3]) : 0u;
#pragma unroll
        for (int ng = 0; ng < 8; ++ng) {
          const int n = nw + ng * 8 + g;
          uint2 b = make_uint2(0u, 0u);
          if (n < N && kin) b = *reinterpret_cast<const uint2*>(Bd + (int64_t)n * r + ka);
          MmaTraits<T>::mma(acc[ng], af, b.x, b.y);
        }
      }
    }
  }
  // c0, c1 = (row g, columns 2 tq, 2 tq + 1), c2, c3 = (row g + 8, same columns) of every 8-column tile
#pragma unroll
  for (int ng = 0; ng < 8; ++ng) {
    const int c = warp * 64 + ng * 8 + 2 * tq;
    *reinterpret_cast<uint32_t*>(tile + g * kExpandRowPad + c) = MmaTraits<T>::pack(acc[ng][0], acc[ng][1]);
    *reinterpret_cast<uint32_t*>(tile + (g + 8) * kExpandRowPad + c) = MmaTraits<T>::pack(acc[ng][2], acc[ng][3]);
  }
  fence_proxy_async_smem();     // the deltas were written by ordinary stores; the bulk copies read them
  __syncthreads();
  if (threadIdx.x < n_tok && s_ids[threadIdx.x] >= 0) {    // one thread per adapter row: one bulk copy each
    const int m = threadIdx.x;
    const uint32_t bytes = (uint32_t)(min(kExpandCols, N - nb) * sizeof(T));
    T* dst = out + (t0 + m) * out_stride + offset + nb;
    if (add) bulk_reduce_add<T>(dst, tile + m * kExpandRowPad, bytes);
    else bulk_store_1d(dst, tile + m * kExpandRowPad, bytes);
    tma_store_commit();
    tma_store_wait_read();      // shared memory must stay until the copy has read it; the grid's end completes the writes
  }
}

template <typename T>
void launch_shrink_mma(float* out, const void* x, int64_t x_stride, const void* A, const int* ids, int64_t T_, int mt, int r,
                       int K, float scale, size_t smem, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    const unsigned grid = (unsigned)((T_ + mt - 1) / mt);
#define B200_SHRINK_CASE(NT_)                                                                                         \
  {                                                                                                                   \
    if (smem > 48 * 1024) ensure_dynamic_smem((const void*)lora_shrink_mma_kernel<T, NT_>, (int)smem);                \
    lora_shrink_mma_kernel<T, NT_><<<grid, 256, smem, st>>>(out, (const T*)x, x_stride, (const T*)A, ids, T_, mt, r, K, scale); \
  }
    if (r <= 8) B200_SHRINK_CASE(1)
    else if (r <= 16) B200_SHRINK_CASE(2)
    else if (r <= 32) B200_SHRINK_CASE(4)
    else B200_SHRINK_CASE(8)
#undef B200_SHRINK_CASE
  }
}

template <typename T>
void launch_expand_mma(dim3 grid, size_t smem, void* out, int64_t out_stride, int offset, const float* h, const void* B,
                       const int* ids, int64_t T_, int N, int r, int add, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    if (smem > 48 * 1024) ensure_dynamic_smem((const void*)lora_expand_mma_kernel<T>, (int)smem);
    lora_expand_mma_kernel<T><<<grid, 256, smem, st>>>((T*)out, out_stride, offset, h, (const T*)B, ids, T_, N, r, add);
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_lora_shrink(float* out, const void* x, int64_t x_stride, const void* A, const int* ids, int64_t T_, int r,
                                int K, float scale, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  int esz = dtype == 0 ? 4 : 2;
  if (K % (16 / esz) != 0 || (x_stride * esz) % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(A) % 16 != 0) return 3;
  const size_t row = (size_t)K * esz;
  if (row > 200 * 1024) return 3;
  if (dtype != 0 && r <= b200::kShrinkMaxRank && K % 32 == 0) {
    // tensor-core form: rows padded by 64 bytes; 8 tokens per tile when they fit in 66 KB (three blocks per SM), else
    // as many as 200 KB hold
    const size_t prow = row + b200::kShrinkRowPad * esz;
    int mt = (int)((66 * 1024) / prow);
    if (mt < b200::kShrinkTile) mt = (int)((200 * 1024) / prow);
    mt = mt < 1 ? 1 : (mt > b200::kShrinkTile ? b200::kShrinkTile : mt);
    const size_t smem = prow * mt + (size_t)8 * 8 * r * 4;
    B200_DISPATCH_DTYPE(dtype, (b200::launch_shrink_mma<T>(out, x, x_stride, A, ids, T_, mt, r, K, scale, smem, st)));
    return cudaGetLastError() != cudaSuccess;
  }
  // tokens per tile: as many as 64 KB of shared memory hold (three blocks per SM), at least one, at most 8
  int mt = (int)((64 * 1024) / row);
  mt = mt < 1 ? 1 : (mt > b200::kShrinkTile ? b200::kShrinkTile : mt);
  const size_t smem = row * mt;
  B200_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024) b200::ensure_dynamic_smem((const void*)b200::lora_shrink_kernel<T>, (int)smem);
    b200::lora_shrink_kernel<T><<<(unsigned)((T_ + mt - 1) / mt), 256, smem, st>>>(out, (const T*)x, x_stride, (const T*)A, ids,
                                                                                  T_, mt, r, K, scale);
  });
  return cudaGetLastError() != cudaSuccess;
}

extern "C" int b200_lora_expand(void* out, int64_t out_stride, int offset, const float* h, const void* B, const int* ids,
                                int64_t T_, int N, int r, int add, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  if ((size_t)r * b200::kExpandTile * 4 > 48 * 1024) return 3;
  const int esz = dtype == 0 ? 4 : 2;
  const int64_t tiles = (T_ + b200::kExpandTile - 1) / b200::kExpandTile;
  // the bulk-copy form needs 16-byte aligned row segments (and B rows that load as whole vectors)
  const bool bulk = reinterpret_cast<uintptr_t>(out) % 16 == 0 && (out_stride * esz) % 16 == 0 && (offset * esz) % 16 == 0 &&
                    (N * esz) % 16 == 0 && (r * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(B) % 16 == 0 && tiles <= 65535;
  if (bulk && dtype != 0 && r % 4 == 0) {   // 16-bit: tensor-core form
    dim3 grid((N + b200::kExpandCols - 1) / b200::kExpandCols, (unsigned)tiles);
    const size_t smem = (size_t)b200::kExpandTile * b200::kExpandRowPad * esz + (size_t)r * b200::kExpandTile * 4;
    B200_DISPATCH_DTYPE(dtype, (b200::launch_expand_mma<T>(grid, smem, out, out_stride, offset, h, B, ids, T_, N, r, add, st)));
    return cudaGetLastError() != cudaSuccess;
  }
  if (bulk) {
    dim3 grid((N + b200::kExpandCols - 1) / b200::kExpandCols, (unsigned)tiles);   // column blocks of a token tile run together
    const size_t smem = (size_t)b200::kExpandTile * b200::kExpandCols * esz + (size_t)r * b200::kExpandTile * 4;
    B200_DISPATCH_DTYPE(dtype, {
      if (smem > 48 * 1024) b200::ensure_dynamic_smem((const void*)b200::lora_expand_bulk_kernel<T>, (int)smem);
      b200::lora_expand_bulk_kernel<T><<<grid, 256, smem, st>>>((T*)out, out_stride, offset, h, (const T*)B, ids, T_, N, r, add);
    });
    return cudaGetLastError() != cudaSuccess;
  }
  dim3 grid((unsigned)tiles, (N + 511) / 512);
  // two adjacent 16-bit columns go out as one 4-byte access when every such pair is 4-byte aligned
  const int pair_ok = (out_stride % 2 == 0 && offset % 2 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0) ? 1 : 0;
  B200_DISPATCH_DTYPE(dtype, (b200::lora_expand_kernel<T><<<grid, 256, (size_t)r * b200::kExpandTile * 4, st>>>(
                                 (T*)out, out_stride, offset, h, (const T*)B, ids, T_, N, r, add, pair_ok)));
  return cudaGetLastError() != cudaSuccess;
}
