// Shared pieces of the paged attention kernels: cp.async / ldmatrix / mma.sync wrappers, the
// XOR-swizzled shared-memory tile layout and the launch parameter block.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "../common/utils.cuh"

namespace b200 {

constexpr int kAttnThreads = 128;
constexpr int kTileN = 64;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

template <typename T> struct MmaTraits;
template <> struct MmaTraits<__nv_bfloat16> {
  __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct MmaTraits<__half> {
  __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// swizzled element offset of 16-byte chunk `chunk` in row `row` of a [rows][D] tile
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
  return row * D + ((chunk ^ (row & 7)) << 3);
}

struct AttnParams {
  const void* q;          // [T, Hq, D]
  const void* kv_cache;   // [blocks, 2, Hkv, bs, D]
  void* out;              // [T, Hq, D]
  float* ws_o;            // [splits, T, Hq, D]   (splits > 1)
  float* ws_lse;          // [splits, T, Hq]
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;      // [B]
  const int* qsl;           // [B+1]
  const float* sinks;       // [Hq] or null
  int Hq, Hkv, block_size, max_blocks, num_splits, window;
  int fuse_merge;         // decode kernel: the last split CTA of a tile merges the partials itself
  int64_t num_blocks, T;
  float scale_log2;
};


// decode-shaped batches (<= 16 packed query rows per KV head): csrc/attention/paged_decode.cu
// *merged is set when the kernel combined its split-KV partials itself (no merge kernel needed)
int paged_decode_dispatch(const AttnParams& p, int B, int max_q_rows, int D, int dtype, cudaStream_t st, bool* merged);

}  // namespace b200
