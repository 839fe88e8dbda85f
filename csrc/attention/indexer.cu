// DeepSeek-V3.2 lightning indexer: fp8 scoring over the paged key cache and per-row top-k.
//
// logits[t, j] = k_scale[j] * sum_h w[t, h] * relu( q[t, h, :] . k[j, :] )      j <= pos(t)
//   q  [T, H=64, 128] e4m3 (per-(token, head) scale folded into w), keys in the page-major cache (per block: rows of 128 e4m3, then f32 scales)
// Keys are the M side of fp8 tensor-core MMAs (mma.sync m16n8k32 e4m3), the 64 heads the N side,
// so the head reduction is a sum along accumulator columns: 16 adds + two quad shuffles per key.
// One CTA = 4 warps scores a 512-key chunk for one query token; the query fragments stay in
// registers.  topk_rows_kernel then selects the k largest logits of each row with a 4-pass radix
// select in shared memory (unordered output, -1 padded).
#include <cuda_fp8.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

constexpr int kIdxH = 64;
constexpr int kIdxD = 128;
constexpr int kIdxChunk = 512;
constexpr int kIdxRow = 132;

__device__ __forceinline__ void mma_e4m3(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
  uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// byte offset of 16-byte chunk `ch` (0..7) of 128-byte row `row`, XOR-swizzled
__device__ __forceinline__ int swz8(int row, int ch) { return row * 128 + ((ch ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(128) indexer_logits_kernel(
    float* __restrict__ logits, const uint8_t* __restrict__ q, const float* __restrict__ w,
    const uint8_t* __restrict__ k_cache, const int* __restrict__ block_tables, const int* __restrict__ seq_lens,
    const int* __restrict__ qsl, const int* __restrict__ req_of_token, int B, int block_size, int max_blocks,
    int64_t total_slots, int64_t ld_logits, int64_t t0) {
  __shared__ __align__(16) uint8_t sQ[kIdxH * kIdxD];
  __shared__ __align__(16) uint8_t sK[4][16 * kIdxD];
  __shared__ float sW[kIdxH];
  __shared__ float sKs[4][16];
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t t = blockIdx.y;
  const int req = req_of_token[t];
  if (req < 0 || req >= B) return;
  const int qs = qsl[req], q_len = qsl[req + 1] - qs;
  // rows are tokens t0 .. t0 + gridDim.y of the batch (a rank may score a slice of the tokens only)
  const int n_keys = seq_lens[req] - q_len + (int)(t + t0 - qs) + 1;
  const int key_lo = blockIdx.x * kIdxChunk;
  float* out = logits + t * ld_logits;
  if (key_lo >= n_keys) {
    for (int j = key_lo + tid; j < min((int64_t)key_lo + kIdxChunk, ld_logits); j += 128) out[j] = -INFINITY;
    return;
  }
  // query: 64 rows of 128 bytes
  for (int c = tid; c < kIdxH * 8; c += 128) {
    int r = c >> 3, ch = c & 7;
    *reinterpret_cast<uint4*>(sQ + swz8(r, ch)) = *reinterpret_cast<const uint4*>(q + (t * kIdxH + r) * kIdxD + ch * 16);
  }
  if (tid < kIdxH) sW[tid] = w[t * kIdxH + tid];
  __syncthreads();
  uint32_t qf[8][4][2];  // [n-tile][k-step][b0, b1]
#pragma unroll
  for (int np = 0; np < 4; ++np) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t r4[4];
      int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
      int ch = ks * 2 + ((lane >> 3) & 1);
      ldsm_x4(r4, sQ + swz8(row, ch));
      qf[2 * np][ks][0] = r4[0]; qf[2 * np][ks][1] = r4[1];
      qf[2 * np + 1][ks][0] = r4[2]; qf[2 * np + 1][ks][1] = r4[3];
    }
  }
  float wa[8][2];  // weights of this thread's accumulator columns
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) { wa[nt][0] = sW[nt * 8 + (lane & 3) * 2]; wa[nt][1] = sW[nt * 8 + (lane & 3) * 2 + 1]; }

  const int* bt = block_tables + (int64_t)req * max_blocks;
  const int chunk_end = min(n_keys, key_lo + kIdxChunk);
  for (int base = key_lo + warp * 16; base < key_lo + kIdxChunk; base += 64) {
    if (base < chunk_end) {
      // 16 key rows: one 128-byte row per iteration, a 4-byte word per lane; word 32 is the scale
#pragma unroll 4
      for (int r = 0; r < 16; ++r) {
        int j = base + r;
        uint32_t word = 0;
        float sc = 0.f;
        if (j < chunk_end) {
          int bi = j / block_size;
          int64_t blk = bi < max_blocks ? bt[bi] : -1;
          int64_t slot = blk >= 0 ? blk * block_size + j % block_size : -1;
          if (slot >= 0 && slot < total_slots) {
            const uint8_t* blkp = k_cache + blk * ((int64_t)block_size * kIdxRow);
            const int off = j % block_size;
            word = reinterpret_cast<const uint32_t*>(blkp + off * kIdxD)[lane];
            if (lane == 0) sc = reinterpret_cast<const float*>(blkp + block_size * kIdxD)[off];
          }
        }
        *reinterpret_cast<uint32_t*>(sK[warp] + swz8(r, lane >> 2) + (lane & 3) * 4) = word;
        if (lane == 0) sKs[warp][r] = sc;
      }
      __syncwarp();
      float acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        ldsm_x4(a, sK[warp] + swz8(row, ks * 2 + (lane >> 4)));
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_e4m3(acc[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
      }
      float la = 0.f, lb = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        la += fmaxf(acc[nt][0], 0.f) * wa[nt][0] + fmaxf(acc[nt][1], 0.f) * wa[nt][1];
        lb += fmaxf(acc[nt][2], 0.f) * wa[nt][0] + fmaxf(acc[nt][3], 0.f) * wa[nt][1];
      }
      la += __shfl_xor_sync(0xffffffff, la, 1); la += __shfl_xor_sync(0xffffffff, la, 2);
      lb += __shfl_xor_sync(0xffffffff, lb, 1); lb += __shfl_xor_sync(0xffffffff, lb, 2);
      if ((lane & 3) == 0) {
        int ra = lane >> 2, rb = ra + 8;
        if (base + ra < ld_logits) out[base + ra] = (base + ra < n_keys) ? la * sKs[warp][ra] : -INFINITY;
        if (base + rb < ld_logits) out[base + rb] = (base + rb < n_keys) ? lb * sKs[warp][rb] : -INFINITY;
      }
      __syncwarp();
    } else {
      for (int j = base + lane; j < base + 16; j += 32)
        if (j < ld_logits) out[j] = -INFINITY;
    }
  }
}

__device__ __forceinline__ uint32_t f2ord(float f) {
  uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One CTA per row: indices of the k largest of logits[row, 0..n), unordered, -1 padded (4-pass radix select on the
// order-preserving 32-bit keys, then two collection passes).  kResident: the row's keys are loaded into shared memory
// once and all six passes run there (rows of up to ~55 K entries); otherwise every pass re-reads the row.
template <bool kResident>
__global__ void __launch_bounds__(512) topk_rows_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                        const int* __restrict__ row_len, int64_t ld, int k,
                                                        int64_t max_len) {
  extern __shared__ uint32_t s_keys[];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_need, s_cnt_gt, s_cnt_eq;
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  const float* x = logits + row * ld;
  int n = row_len ? row_len[row] : (int)max_len;
  if (n > max_len) n = (int)max_len;
  int* o = out + row * (int64_t)k;
  const int tid = threadIdx.x;
  if (n <= k) {
    for (int i = tid; i < k; i += 512) o[i] = i < n ? i : -1;
    return;
  }
  if (tid == 0) { s_prefix = 0; s_mask = 0; s_need = k; }
  if (kResident) {
    int i = tid * 4;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      for (; i + 3 < n; i += 512 * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        s_keys[i] = f2ord(v.x); s_keys[i + 1] = f2ord(v.y); s_keys[i + 2] = f2ord(v.z); s_keys[i + 3] = f2ord(v.w);
      }
      for (int j = (n & ~3) + tid; j < n; j += 512) s_keys[j] = f2ord(x[j]);
    } else {
      for (int j = tid; j < n; j += 512) s_keys[j] = f2ord(x[j]);
    }
  }
  auto key = [&](int i) -> uint32_t { return kResident ? s_keys[i] : f2ord(x[i]); };
  __syncthreads();
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = tid; i < 256; i += 512) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    const int shift = pass * 8;
    for (int i = tid; i < n; i += 512) {
      uint32_t u = key(i);
      if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, acc = 0, b = 255;
      for (; b > 0; --b) {
        if (acc + hist[b] >= need) break;
        acc += hist[b];
      }
      s_need = need - acc;  // how many to take from bin b (with the longer prefix)
      s_prefix = prefix | ((uint32_t)b << shift);
      s_mask = mask | (255u << shift);
    }
    __syncthreads();
  }
  // threshold value = s_prefix (exact 32-bit key); take all greater, and s_need of the equal ones
  const uint32_t thr = s_prefix;
  const int need_eq = s_need;
  if (tid == 0) { s_cnt_gt = 0; s_cnt_eq = 0; }
  __syncthreads();
  for (int i = tid; i < n; i += 512) {
    uint32_t u = key(i);
    if (u > thr) {
      int p = atomicAdd(&s_cnt_gt, 1);
      if (p < k) o[p] = i;
    }
  }
  __syncthreads();
  const int base = s_cnt_gt;
  for (int i = tid; i < n; i += 512) {
    uint32_t u = key(i);
    if (u == thr) {
      int p = atomicAdd(&s_cnt_eq, 1);
      if (p < need_eq && base + p < k) o[base + p] = i;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_indexer_logits(float* logits, const void* q_fp8, const float* w, const void* k_cache,
                                   const int* block_tables, const int* seq_lens, const int* qsl,
                                   const int* req_of_token, int64_t T_, int B, int block_size, int max_blocks,
                                   int64_t total_slots, int64_t ld_logits, int64_t t0, cudaStream_t st) {
  if (T_ == 0) return 0;
  dim3 grid((unsigned)((ld_logits + kIdxChunk - 1) / kIdxChunk), (unsigned)T_);
  return (int)launch_pdl(indexer_logits_kernel, grid, dim3(128), 0, st, logits, (const uint8_t*)q_fp8, w,
                         (const uint8_t*)k_cache, block_tables, seq_lens, qsl, req_of_token, B, block_size, max_blocks,
                         total_slots, ld_logits, t0);
}

extern "C" int b200_topk_rows(int* out, const float* logits, const int* row_len, int64_t rows, int64_t ld, int k,
                              int64_t max_len, cudaStream_t st) {
  if (rows == 0) return 0;
  // rows of up to 220 KB of keys stay resident in shared memory for all six passes
  const int64_t bytes = max_len * 4;
  if (bytes <= 220 * 1024) {
    auto kern = topk_rows_kernel<true>;
    cudaError_t e = ensure_dynamic_smem((const void*)kern, 220 * 1024);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(kern, dim3((unsigned)rows), dim3(512), (size_t)bytes, st, out, logits, row_len, ld, k, max_len);
  }
  return (int)launch_pdl(topk_rows_kernel<false>, dim3((unsigned)rows), dim3(512), 0, st, out, logits, row_len, ld, k,
                         max_len);
}
