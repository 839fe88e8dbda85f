// Rotary embedding and KV-cache movement kernels.
//
// Cache layouts (see vllm_kunlun_b200/ops/reference/attention.py):
//   GQA     kv_cache[block][2][kv_head][slot_in_block][head_dim]
//   MLA     kv_cache[block][slot_in_block][576]   (bf16) or uint8 [..][656] (512 e4m3 | 4 f32 | 64 bf16)
//   indexer k_cache[block]: block_size rows of 128 e4m3 bytes, then block_size f32 scales (132 bytes per slot)
// Slot ids < 0 mark padding rows and are skipped.  Every index read from a table is range-checked
// against the tensor bounds before it is used as an address.
#include <cuda_fp8.h>
#include <math.h>

#include "../api.h"
#include "../common/launch.cuh"
#include "../common/utils.cuh"

namespace b200 {

__device__ __forceinline__ void rope_pair(float& a, float& b, float c, float s) {
  float x = a, y = b;
  a = x * c - y * s;
  b = y * c + x * s;
}

// One warp per (token, head).  Heads [0, Hq) are queries, [Hq, Hq+Hkv) keys, the rest values.
template <typename T>
__global__ void qkv_split_norm_rope_cache_kernel(
    T* __restrict__ q_out, const T* __restrict__ qkv, const int64_t* __restrict__ positions,
    const float* __restrict__ cos_sin, const T* __restrict__ q_w, const T* __restrict__ k_w, float eps, int Hq,
    int Hkv, int D, int rot_dim, int neox, int gemma, T* __restrict__ kv_cache, const int64_t* __restrict__ slots,
    int block_size, int64_t num_blocks, int64_t max_pos, int64_t qkv_stride) {
  extern __shared__ float sm[];
  griddep_launch();
  griddep_wait();
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x;
  const int head = blockIdx.y * warps + wid;
  const int total_heads = Hq + 2 * Hkv;
  if (head >= total_heads) return;
  float* buf = sm + wid * D;
  const T* src = qkv + t * qkv_stride + (int64_t)head * D;
  const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
  for (int i = lane; i < D; i += 32) buf[i] = to_f(src[i]);
  __syncwarp();
  if (is_q || is_k) {
    const T* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss += buf[i] * buf[i];
      ss = warp_sum(ss);
      float inv = rsqrtf(ss / D + eps);
      // round to T between norm and rotary, as two separate kernels would
      for (int i = lane; i < D; i += 32) buf[i] = to_f(from_f<T>(buf[i] * inv * (to_f(w[i]) + (gemma ? 1.f : 0.f))));
      __syncwarp();
    }
    int64_t pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + pos * rot_dim;
    const int half = rot_dim >> 1;
    for (int j = lane; j < half; j += 32) {
      float c = cs[j], s = cs[half + j];
      if (neox) rope_pair(buf[j], buf[j + half], c, s);
      else rope_pair(buf[2 * j], buf[2 * j + 1], c, s);
    }
    __syncwarp();
  }
  if (is_q) {
    T* dst = q_out + (t * Hq + head) * (int64_t)D;
    for (int i = lane; i < D; i += 32) dst[i] = from_f<T>(buf[i]);
  } else if (kv_cache != nullptr) {
    int64_t slot = slots[t];
    if (slot < 0 || slot >= num_blocks * block_size) return;
    int kvh = is_k ? head - Hq : head - Hq - Hkv;
    int64_t blk = slot / block_size, off = slot % block_size;
    T* dst = kv_cache + ((((blk * 2 + (is_k ? 0 : 1)) * Hkv + kvh) * block_size + off) * (int64_t)D);
    for (int i = lane; i < D; i += 32) dst[i] = from_f<T>(buf[i]);
  }
}

// In-place rotary on separate q [T, Hq*D] and k [T, Hk*D] (rows may be strided).
template <typename T>
__global__ void rope_kernel(T* __restrict__ q, T* __restrict__ k, const int64_t* __restrict__ positions,
                            const float* __restrict__ cos_sin, int Hq, int Hk, int D, int rot_dim, int neox,
                            int64_t max_pos, int64_t q_stride, int64_t k_stride, const int64_t* positions3,
                            int sec0, int sec1, int interleaved, int64_t T_) {
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x;
  const int head = blockIdx.y * warps + wid;
  if (head >= Hq + Hk) return;
  T* p = head < Hq ? q + t * q_stride + (int64_t)head * D : k + t * k_stride + (int64_t)(head - Hq) * D;
  const int half = rot_dim >> 1;
  for (int j = lane; j < half; j += 32) {
    int64_t pos;
    if (positions3 != nullptr) {  // M-RoPE: frequency slot j takes the temporal / height / width position
      int axis;
      if (interleaved) axis = (j % 3 == 1 && j < sec1 * 3) ? 1 : ((j % 3 == 2 && j < (rot_dim / 2 - sec0 - sec1) * 3) ? 2 : 0);
      else axis = j < sec0 ? 0 : (j < sec0 + sec1 ? 1 : 2);
      pos = positions3[axis * T_ + t];
    } else {
      pos = positions[t];
    }
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + pos * rot_dim;
    float c = cs[j], s = cs[half + j];
    int ia = neox ? j : 2 * j, ib = neox ? j + half : 2 * j + 1;
    float a = to_f(p[ia]), b = to_f(p[ib]);
    rope_pair(a, b, c, s);
    p[ia] = from_f<T>(a);
    p[ib] = from_f<T>(b);
  }
}

template <typename T>
__global__ void reshape_and_cache_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ kv_cache,
                                         const int64_t* __restrict__ slots, int Hkv, int D, int block_size,
                                         int64_t num_blocks, int64_t k_stride, int64_t v_stride) {
  const int64_t t = blockIdx.x;
  int64_t slot = slots[t];
  if (slot < 0 || slot >= num_blocks * block_size) return;
  int64_t blk = slot / block_size, off = slot % block_size;
  for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
    int h = i / D, d = i % D;
    kv_cache[(((blk * 2 + 0) * Hkv + h) * block_size + off) * (int64_t)D + d] = k[t * k_stride + i];
    kv_cache[(((blk * 2 + 1) * Hkv + h) * block_size + off) * (int64_t)D + d] = v[t * v_stride + i];
  }
}

template <typename T>
__global__ void concat_and_cache_mla_kernel(const T* __restrict__ kv_c, const T* __restrict__ k_pe,
                                            T* __restrict__ cache, const int64_t* __restrict__ slots, int rank,
                                            int rope, int64_t total_slots, int64_t kvc_stride, int64_t kpe_stride) {
  const int64_t t = blockIdx.x;
  int64_t slot = slots[t];
  if (slot < 0 || slot >= total_slots) return;
  T* dst = cache + slot * (int64_t)(rank + rope);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = kv_c[t * kvc_stride + i];
  for (int i = threadIdx.x; i < rope; i += blockDim.x) dst[rank + i] = k_pe[t * kpe_stride + i];
}

__device__ __forceinline__ float from_e4m3(uint8_t b) {
  __nv_fp8_e4m3 q;
  q.__x = b;
  return static_cast<float>(q);
}
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// 656-byte rows: 4 x (128 e4m3) | 4 x f32 scale | 64 bf16.  One block of 128 threads per token:
// warp g quantises group g.
template <typename T>
__global__ void __launch_bounds__(128) concat_and_cache_mla_fp8_kernel(
    const T* __restrict__ kv_c, const T* __restrict__ k_pe, uint8_t* __restrict__ cache,
    const int64_t* __restrict__ slots, int64_t total_slots, int64_t kvc_stride, int64_t kpe_stride) {
  const int64_t t = blockIdx.x;
  int64_t slot = slots[t];
  if (slot < 0 || slot >= total_slots) return;
  uint8_t* row = cache + slot * 656;
  int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = to_f(kv_c[t * kvc_stride + g * 128 + lane * 4 + j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = fmaxf(warp_max(amax), 1e-10f);
  float scale = amax / 448.f;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= (uint32_t)to_e4m3(v[j] / scale) << (8 * j);
  reinterpret_cast<uint32_t*>(row)[g * 32 + lane] = packed;
  if (lane == 0) reinterpret_cast<float*>(row + 512)[g] = scale;
  if (threadIdx.x < 64) reinterpret_cast<__nv_bfloat16*>(row + 528)[threadIdx.x] =
      __float2bfloat16(to_f(k_pe[t * kpe_stride + threadIdx.x]));
}

// Page-major indexer cache: a block holds its key rows (128 e4m3 each) first and their f32 scales (powers of two
// when ue8m0) after them, so that a page of keys is one contiguous 16-byte aligned tile.  One warp per token.
template <typename T>
__global__ void indexer_k_quant_and_cache_kernel(const T* __restrict__ k, uint8_t* __restrict__ cache,
                                                 const int64_t* __restrict__ slots, int64_t T_, int64_t total_slots,
                                                 int ue8m0, int64_t k_stride, int block_size) {
  int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  int lane = threadIdx.x & 31;
  int64_t slot = slots[t];
  if (slot < 0 || slot >= total_slots) return;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = to_f(k[t * k_stride + lane * 4 + j]); amax = fmaxf(amax, fabsf(v[j])); }
  amax = fmaxf(warp_max(amax), 1e-10f);
  float scale = amax / 448.f;
  if (ue8m0) scale = exp2f(ceilf(log2f(scale)));
  uint8_t* blk = cache + (slot / block_size) * ((int64_t)block_size * 132);
  const int off = (int)(slot % block_size);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= (uint32_t)to_e4m3(v[j] / scale) << (8 * j);
  reinterpret_cast<uint32_t*>(blk + off * 128)[lane] = packed;
  if (lane == 0) reinterpret_cast<float*>(blk + block_size * 128)[off] = scale;
}

// Lightning-indexer operand preparation in one launch (the reference runs it as separate layer-norm, rotary,
// concatenation, quantisation and cache-write ops, models/deepseek_v2.py:661-788).  One CTA per token, 8 warps:
//   * every (token, head) row of q [T, H, 128]: rotary (neox halves) on the leading 64 dims, rounded to the
//     activation type as the unfused path does, then e4m3 with one power-of-two scale per row;
//     w[t, h] = head_weight[t, h] * wscale * q_scale  (what the logits kernel multiplies a head's ReLU'd score with);
//   * the token's key k [T, 128]: LayerNorm (fp32 statistics, weight + bias), rotary on the leading 64 dims, e4m3 +
//     scale into the page-major indexer cache (key rows first, scales after them in every block).
// Lane l owns dims 4l .. 4l + 3; a rotary pair (d, d + 32) sits in lanes l and l ^ 8 (l < 16).
template <typename T>
__global__ void indexer_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ ln_w,
                                    const T* __restrict__ ln_b, const int64_t* __restrict__ positions,
                                    const float* __restrict__ cos_sin, const T* __restrict__ head_w, float wscale,
                                    uint8_t* __restrict__ q_out, float* __restrict__ w_out, uint8_t* __restrict__ cache,
                                    const int64_t* __restrict__ slots, int H, int64_t max_pos, int64_t total_slots,
                                    int64_t q_stride, int64_t k_stride, int64_t hw_stride, float eps, int ue8m0,
                                    int64_t q_lo, int64_t q_hi, int block_size) {
  // q / head_w / q_out / w_out hold tokens [q_lo, q_hi) only (a rank may score a slice of the batch); keys: all tokens
  constexpr int kRot = 64, kHalf = 32;
  const int64_t t = blockIdx.x;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  int64_t pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* cs = cos_sin + pos * kRot;
  // this lane's rotary coefficients: dims 4l.. of the first half use frequency slot d, of the second half d - 32
  float c4[4], s4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane * 4 + j;
    const int f = d < kHalf ? d : d - kHalf;
    c4[j] = d < kRot ? cs[f] : 1.f;
    s4[j] = d < kRot ? cs[kHalf + f] : 0.f;
  }
  auto rotate = [&](float (&v)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 8);
      // first half: a' = a c - b s (b = partner); second half: b' = b c + a s (a = partner)
      const float r = lane < 8 ? v[j] * c4[j] - other * s4[j] : v[j] * c4[j] + other * s4[j];
      if (lane < 16) v[j] = to_f(from_f<T>(r));
    }
  };
  auto quantise = [&](const float (&v)[4], float& scale) -> uint32_t {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(warp_max(amax), 1e-10f);
    scale = amax / 448.f;
    if (ue8m0) scale = exp2f(ceilf(log2f(scale)));
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= (uint32_t)to_e4m3(v[j] / scale) << (8 * j);
    return packed;
  };
  for (int h = wid; h <= H; h += warps) {
    float v[4];
    if (h < H) {
      if (t < q_lo || t >= q_hi) continue;
      const int64_t tq = t - q_lo;
      const T* src = q + tq * q_stride + (int64_t)h * 128 + lane * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_f(src[j]);
      rotate(v);
      float scale;
      const uint32_t packed = quantise(v, scale);
      reinterpret_cast<uint32_t*>(q_out + (tq * H + h) * 128)[lane] = packed;
      if (lane == 0) w_out[tq * H + h] = to_f(head_w[tq * hw_stride + h]) * wscale * scale;
    } else {
      const int64_t slot = slots[t];
      if (slot < 0 || slot >= total_slots) continue;
      const T* src = k + t * k_stride + lane * 4;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { v[j] = to_f(src[j]); sum += v[j]; }
      const float mean = warp_sum(sum) * (1.f / 128.f);
      float var = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float d = v[j] - mean; var += d * d; }
      const float rstd = rsqrtf(warp_sum(var) * (1.f / 128.f) + eps);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v[j] = to_f(from_f<T>((v[j] - mean) * rstd * to_f(ln_w[lane * 4 + j]) + to_f(ln_b[lane * 4 + j])));
      rotate(v);
      float scale;
      const uint32_t packed = quantise(v, scale);
      uint8_t* blk = cache + (slot / block_size) * ((int64_t)block_size * 132);
      const int off = (int)(slot % block_size);
      reinterpret_cast<uint32_t*>(blk + off * 128)[lane] = packed;
      if (lane == 0) reinterpret_cast<float*>(blk + block_size * 128)[off] = scale;
    }
  }
}

__global__ void convert_req_index_kernel(int32_t* __restrict__ out, const int32_t* __restrict__ req_id,
                                         const int32_t* __restrict__ block_table, const int32_t* __restrict__ idx,
                                         int64_t T_, int topk, int block_size, int max_blocks, int num_reqs) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T_ * topk) return;
  int64_t t = i / topk;
  int v = idx[i];
  int r = req_id[t];
  int o = -1;
  if (v >= 0 && r >= 0 && r < num_reqs) {
    int b = v / block_size;
    if (b < max_blocks) o = block_table[(int64_t)r * max_blocks + b] * block_size + v % block_size;
  }
  out[i] = o;
}

__global__ void copy_blocks_kernel(uint4* __restrict__ cache, const int64_t* __restrict__ src,
                                   const int64_t* __restrict__ dst, int64_t vec_per_block, int64_t num_blocks) {
  int64_t s = src[blockIdx.x], d = dst[blockIdx.x];
  if (s < 0 || d < 0 || s >= num_blocks || d >= num_blocks) return;
  for (int64_t i = threadIdx.x; i < vec_per_block; i += blockDim.x) cache[d * vec_per_block + i] = cache[s * vec_per_block + i];
}

// out = merge of two partial attention results by log-sum-exp.  o [T,H,D], lse [T,H].
template <typename T>
__global__ void merge_attn_states_kernel(T* __restrict__ out, float* __restrict__ lse_out, const T* __restrict__ o1,
                                         const float* __restrict__ lse1, const T* __restrict__ o2,
                                         const float* __restrict__ lse2, int64_t rows, int D) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int lane = threadIdx.x & 31;
  float a = lse1[row], b = lse2[row];
  float m = fmaxf(a, b);
  if (isinf(m)) m = 0.f;
  float w1 = __expf(a - m), w2 = __expf(b - m);
  float den = fmaxf(w1 + w2, 1e-30f);
  for (int i = lane; i < D; i += 32)
    out[row * D + i] = from_f<T>((to_f(o1[row * D + i]) * w1 + to_f(o2[row * D + i]) * w2) / den);
  if (lane == 0 && lse_out != nullptr) lse_out[row] = m + __logf(den);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_qkv_split_norm_rope_cache(void* q_out, const void* qkv, const int64_t* positions,
                                               const float* cos_sin, const void* q_w, const void* k_w, float eps,
                                               int64_t T_, int Hq, int Hkv, int D, int rot_dim, int neox, int gemma,
                                               void* kv_cache, const int64_t* slots, int block_size,
                                               int64_t num_blocks, int64_t max_pos, int64_t qkv_stride, int dtype,
                                               cudaStream_t st) {
  if (T_ == 0) return 0;
  const int warps = 4;
  dim3 grid((unsigned)T_, (Hq + 2 * Hkv + warps - 1) / warps);
  B200_DISPATCH_DTYPE(dtype, {
    launch_pdl(qkv_split_norm_rope_cache_kernel<T>, grid, dim3(warps * 32), warps * D * sizeof(float), st,
        (T*)q_out, (const T*)qkv, positions, cos_sin, (const T*)q_w, (const T*)k_w, eps, Hq, Hkv, D, rot_dim, neox,
        gemma, (T*)kv_cache, slots, block_size, num_blocks, max_pos, qkv_stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_rope(void* q, void* k, const int64_t* positions, const float* cos_sin, int64_t T_, int Hq, int Hk,
                         int D, int rot_dim, int neox, int64_t max_pos, int64_t q_stride, int64_t k_stride,
                         const int64_t* positions3, int sec0, int sec1, int interleaved, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  const int warps = 4;
  dim3 grid((unsigned)T_, (Hq + Hk + warps - 1) / warps);
  B200_DISPATCH_DTYPE(dtype, {
    rope_kernel<T><<<grid, warps * 32, 0, st>>>((T*)q, (T*)k, positions, cos_sin, Hq, Hk, D, rot_dim, neox, max_pos,
                                               q_stride, k_stride, positions3, sec0, sec1, interleaved, T_);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_reshape_and_cache(const void* k, const void* v, void* kv_cache, const int64_t* slots, int64_t T_,
                                      int Hkv, int D, int block_size, int64_t num_blocks, int64_t k_stride,
                                      int64_t v_stride, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    reshape_and_cache_kernel<T><<<T_, 256, 0, st>>>((const T*)k, (const T*)v, (T*)kv_cache, slots, Hkv, D, block_size,
                                                   num_blocks, k_stride, v_stride);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_concat_and_cache_mla(const void* kv_c, const void* k_pe, void* cache, const int64_t* slots,
                                         int64_t T_, int rank, int rope, int64_t total_slots, int64_t kvc_stride,
                                         int64_t kpe_stride, int fp8, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    if (fp8) {
      if (rank != 512 || rope != 64) return 2;
      concat_and_cache_mla_fp8_kernel<T><<<T_, 128, 0, st>>>((const T*)kv_c, (const T*)k_pe, (uint8_t*)cache, slots,
                                                            total_slots, kvc_stride, kpe_stride);
    } else {
      concat_and_cache_mla_kernel<T><<<T_, 128, 0, st>>>((const T*)kv_c, (const T*)k_pe, (T*)cache, slots, rank, rope,
                                                        total_slots, kvc_stride, kpe_stride);
    }
  });
  return (int)cudaGetLastError();
}

// Gather rows of the paged MLA latent cache by global slot index into a dense 16-bit buffer, de-quantising the
// 656-byte fp8 rows (4 x 128 e4m3 | 4 f32 scales | 64 bf16 rope dims) on the way - the read side of the `fp8_ds_mla`
// cache and the chunk gather of a bounded-workspace prefill context (`gather_and_maybe_dequant_cache`,
// v1/attention/backends/mla/common.py:1557-1612 of the reference).  One warp per output row; a negative or
// out-of-range slot gives a zero row.
template <typename T, bool kFp8>
__global__ void gather_mla_rows_kernel(T* __restrict__ out, const uint8_t* __restrict__ cache,
                                       const int32_t* __restrict__ slots, int64_t M, int64_t total_slots) {
  const int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const int lane = threadIdx.x & 31;
  const int64_t slot = slots[m];
  T* dst = out + m * 576;
  if (slot < 0 || slot >= total_slots) {
    for (int i = lane; i < 576 / 2; i += 32) reinterpret_cast<uint32_t*>(dst)[i] = 0u;
    return;
  }
  if (kFp8) {
    const uint8_t* row = cache + slot * 656;
    const float* sc = reinterpret_cast<const float*>(row + 512);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t w = reinterpret_cast<const uint32_t*>(row)[g * 32 + lane];
      const float s = sc[g];
      T v4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v4[j] = from_f<T>(from_e4m3((uint8_t)(w >> (8 * j))) * s);
      *reinterpret_cast<uint2*>(dst + g * 128 + lane * 4) = *reinterpret_cast<const uint2*>(v4);
    }
    // rope dims are stored as bf16
    const __nv_bfloat16* pe = reinterpret_cast<const __nv_bfloat16*>(row + 528);
    for (int i = lane; i < 64; i += 32) dst[512 + i] = from_f<T>(__bfloat162float(pe[i]));
  } else {
    const uint32_t* row = reinterpret_cast<const uint32_t*>(cache + slot * (576 * sizeof(T)));
    for (int i = lane; i < 576 / 2; i += 32) reinterpret_cast<uint32_t*>(dst)[i] = row[i];
  }
}

extern "C" int b200_gather_mla_rows(void* out, const void* cache, const int32_t* slots, int64_t M, int64_t total_slots,
                                    int fp8, int dtype, cudaStream_t st) {
  if (M == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    if (fp8) gather_mla_rows_kernel<T, true><<<(unsigned)((M + 7) / 8), 256, 0, st>>>((T*)out, (const uint8_t*)cache, slots, M, total_slots);
    else gather_mla_rows_kernel<T, false><<<(unsigned)((M + 7) / 8), 256, 0, st>>>((T*)out, (const uint8_t*)cache, slots, M, total_slots);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_indexer_k_quant_and_cache(const void* k, void* cache, const int64_t* slots, int64_t T_,
                                              int64_t total_slots, int ue8m0, int64_t k_stride, int block_size,
                                              int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    indexer_k_quant_and_cache_kernel<T><<<(T_ + 3) / 4, 128, 0, st>>>((const T*)k, (uint8_t*)cache, slots, T_,
                                                                     total_slots, ue8m0, k_stride, block_size);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_indexer_prep(const void* q, const void* k, const void* ln_w, const void* ln_b, const int64_t* positions,
                                 const float* cos_sin, const void* head_w, float wscale, void* q_out, float* w_out,
                                 void* cache, const int64_t* slots, int64_t T_, int H, int64_t max_pos,
                                 int64_t total_slots, int64_t q_stride, int64_t k_stride, int64_t hw_stride, float eps,
                                 int ue8m0, int64_t q_lo, int64_t q_hi, int block_size, int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    indexer_prep_kernel<T><<<T_, 256, 0, st>>>((const T*)q, (const T*)k, (const T*)ln_w, (const T*)ln_b, positions, cos_sin,
                                               (const T*)head_w, wscale, (uint8_t*)q_out, w_out, (uint8_t*)cache, slots, H,
                                               max_pos, total_slots, q_stride, k_stride, hw_stride, eps, ue8m0, q_lo, q_hi,
                                               block_size);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_convert_req_index(int32_t* out, const int32_t* req_id, const int32_t* block_table,
                                      const int32_t* idx, int64_t T_, int topk, int block_size, int max_blocks,
                                      int num_reqs, cudaStream_t st) {
  int64_t n = T_ * topk;
  if (n == 0) return 0;
  convert_req_index_kernel<<<(n + 255) / 256, 256, 0, st>>>(out, req_id, block_table, idx, T_, topk, block_size,
                                                           max_blocks, num_reqs);
  return (int)cudaGetLastError();
}

extern "C" int b200_copy_blocks(void* cache, const int64_t* src, const int64_t* dst, int64_t n_pairs,
                                int64_t bytes_per_block, int64_t num_blocks, cudaStream_t st) {
  if (n_pairs == 0) return 0;
  if (bytes_per_block % 16) return 2;
  copy_blocks_kernel<<<n_pairs, 256, 0, st>>>((uint4*)cache, src, dst, bytes_per_block / 16, num_blocks);
  return (int)cudaGetLastError();
}

extern "C" int b200_merge_attn_states(void* out, float* lse_out, const void* o1, const float* lse1, const void* o2,
                                      const float* lse2, int64_t rows, int D, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_DISPATCH_DTYPE(dtype, {
    merge_attn_states_kernel<T><<<(rows + 7) / 8, 256, 0, st>>>((T*)out, lse_out, (const T*)o1, lse1, (const T*)o2,
                                                               lse2, rows, D);
  });
  return (int)cudaGetLastError();
}
