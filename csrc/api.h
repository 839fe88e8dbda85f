// C ABI of the sm_100a kernel library.  Kernel sources include only this header and CUDA headers
// (no libtorch), so they compile in seconds; bindings.cpp adapts torch tensors to these calls.
// Every launcher returns 0 on success, a cudaError_t value or a small positive code on bad arguments.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dtype codes: 0 = float32, 1 = bfloat16, 2 = float16

// ---- GEMM (tcgen05) -------------------------------------------------------------------------
typedef struct GemmArgs {
  void* out;          // [T, ldo] bf16/fp16
  const void* bias;   // [N] or null
  float* ws;          // stream-K partial tiles (tiles * max_contrib * bn * 128 floats)
  int* counters;      // per-tile arrival tickets, zero on entry, zero again on exit
  int* status;        // device status word: 0 = ok, otherwise the code of the wait that timed out
  int T, N, K;
  int n_tiles, t_tiles;
  int per_cta;        // stream-K: k-block units per CTA; 0 = whole tiles, strided over the grid
  int max_contrib;    // stream-K: workspace slots per tile
  int grid;
  int fmt;            // 1 = bf16, 0 = fp16
  int ldo;            // row stride of out (elements)
  int bn;             // token tile: 16 / 32 / 64 / 128 / 256
  int num_sms;
  int stages;         // 0 = choose from the shared-memory budget
  int ctas_per_sm;    // 0 = choose (2 for small token tiles)
  int act;            // 0 = plain; 1 silu, 2 gelu-tanh, 3 swigluoai on [64 gate | 64 up] interleaved weight tiles
  // collective fusion over peer memory (all zero / null = plain GEMM)
  void* rs_stage[8];  // reduce-scatter: staging area of every rank (peer mappings)
  void* rs_flags[8];  // reduce-scatter: per-(source, token tile) arrival counters on every rank
  const void* ag_flags;  // all-gather: local per-token-tile arrival counters
  int rs_on, rs_tloc, rs_rank, ag_on, ag_expect;
  unsigned spin_limit;
  // signed 8-bit operands (kind::i8): per-token activation scales [T], per-channel weight scales [N]; fmt = output type
  int i8;
  const float* a_scale;
  const float* w_scale;
} GemmArgs;
int b200_gemm_pick_bn(int T);
int b200_gemm_launch(const GemmArgs* a, const void* tmapW, const void* tmapX, cudaStream_t st);

// Decode-sized GEMM (one token tile of at most 32 rows): cluster split-K with the reduction in the leader CTA's
// shared memory; optional gated activation or tensor-parallel push epilogue (gemm/gemm_decode.cu).
typedef struct GemmDecodeArgs {
  void* out;            // [T, ldo]
  const void* bias;     // [N] or null
  int* status;
  int T, N, K;
  int n_tiles;          // ceil(N / 128)
  int S;                // CTAs per cluster = K splits per weight tile, 1..8 (at most 4 when bn = 32)
  int kb_per_cta;       // ceil(ceil(K / 64) / S); (S - 1) * kb_per_cta must be < ceil(K / 64)
  int fmt, ldo, bn;     // bn: 16 or 32
  int stages;           // 0 = choose
  int ctas_per_sm;      // 1 or 2: shared-memory budget per CTA
  int act;              // as in GemmArgs
  // row-parallel epilogue under tensor parallelism: store locally and push {data, epoch} units to every peer
  int ar_on, rank, nranks;
  void* ll_bufs[8];     // low-latency all-reduce buffers of all ranks (peer mappings)
  const void* epoch_word;  // device word holding the number of completed all-reduce calls
  int64_t ll_slot_bytes;
  // fp8 e4m3 operands with 128x128 weight block scales and 1x128 activation scales (fmt then names the output type;
  // a k-block is 128 elements, so kb_per_cta counts blocks of 128)
  int fp8;
  const float* a_scale;    // [ceil(K/128), a_stride] transposed activation scales
  const float* w_scale;    // [ceil(N/128), ceil(K/128)]
  int a_stride;
  int i8;  // signed 8-bit operands (kind::i8): a_scale [T] per token, w_scale [N] per channel; fmt = output type
  // 4-bit weights (AWQ / GPTQ after repacking): the weight tensor map covers the packed bytes [N, K / 2] (32-byte x
  // 128-row boxes, no swizzle); scale / zero [N, K / group] in the activation type; group a multiple of 64
  int w4, w4_group;
  const void* w4_scale;
  const void* w4_zero;
  // qkv epilogue (head_dim 128): split + optional q / k RMSNorm + rotary + K / V cache write; out = q [T, Hq * 128]
  int qk_on, qk_hq, qk_hkv, qk_neox, qk_gemma, qk_block_size;
  float qk_eps;
  const int64_t* qk_positions;
  const float* qk_cos_sin;
  const void* qk_q_w;
  const void* qk_k_w;
  void* qk_kv_cache;
  const int64_t* qk_slots;
  int64_t qk_num_blocks, qk_max_pos;
} GemmDecodeArgs;
int b200_gemm_decode_launch(const GemmDecodeArgs* a, const void* tmapW, const void* tmapX, cudaStream_t st);

// Grouped (rows sorted by expert) and/or fp8 block-scaled GEMM; lod == null -> one group of M rows.
typedef struct GroupedGemmArgs {
  void* out;             // [M, ldo] bf16/fp16
  const void* bias;      // [E, N] or null
  const int* lod;        // [E + 1] device, or null
  const float* a_scale;  // fp8: [ceil(K/128), a_stride] transposed activation scales
  const float* w_scale;  // fp8: [E, ceil(N/128), ceil(K/128)]
  int* status;
  int M, N, K, E, ldo, a_stride;
  int fp8;               // 1 = e4m3 inputs
  int fmt;               // 16-bit inputs: 1 = bf16, 0 = fp16
  int out_fmt;           // 1 = bf16, 0 = fp16
  int bn;                // token tile 16 / 32 / 64 / 128
  int grid;
} GroupedGemmArgs;
int b200_grouped_gemm_launch(const GroupedGemmArgs* a, const void* tmapW, const void* tmapX, cudaStream_t st);

// Encodes a 2-D row-major [rows, cols] tensor map with a [box_rows, box_cols] box and 128-byte
// swizzle into `out` (128 bytes).  elem_bytes = 1 or 2.
int b200_encode_tmap_2d(void* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                        uint32_t box_rows, uint32_t box_cols, int elem_bytes);

// Same for a plain (unswizzled) byte tensor: [rows, row_bytes] with a [box_rows, box_bytes] box; box_bytes a multiple
// of 16.
int b200_encode_tmap_2d_raw(void* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t row_stride_bytes,
                            uint32_t box_rows, uint32_t box_bytes);
// out [N, K] (bf16 / fp16) = (q - zero) * scale of 4-bit weights packed as [N, K / 2] (see quantization/int4.py)
int b200_dequant_w4(void* out, const void* packed, const void* scale, const void* zero, int64_t N, int K, int group,
                    int dtype, cudaStream_t st);

// ---- elementwise ----------------------------------------------------------------------------
int b200_rmsnorm(void* out, const void* x, void* residual, const void* w, int64_t rows, int H, float eps, int gemma,
                 int64_t x_stride, int64_t out_stride, int dtype, cudaStream_t st);
int b200_rownorm(void* out, const void* x, const void* z, const void* w, int64_t rows, int D, float eps, int mode,
                 int dtype, cudaStream_t st);
int b200_act_and_mul(void* out, const void* x, int64_t rows, int d, int act, int dtype, cudaStream_t st);
int b200_quick_gelu(void* out, const void* x, int64_t n, int dtype, cudaStream_t st);
int b200_embedding(void* out, const int64_t* ids, const void* w, int64_t T, int H, int64_t rows, int64_t vocab_start,
                   int dtype, cudaStream_t st);
// scratch_val / scratch_idx: rows * chunks entries each (partial maxima)
int b200_argmax(int64_t* out, const void* logits, int64_t rows, int V, int64_t stride, int dtype, float* scratch_val,
                int* scratch_idx, int chunks, cudaStream_t st);

// ---- rotary / cache -------------------------------------------------------------------------
int b200_qkv_split_norm_rope_cache(void* q_out, const void* qkv, const int64_t* positions, const float* cos_sin,
                                   const void* q_w, const void* k_w, float eps, int64_t T, int Hq, int Hkv, int D,
                                   int rot_dim, int neox, int gemma, void* kv_cache, const int64_t* slots,
                                   int block_size, int64_t num_blocks, int64_t max_pos, int64_t qkv_stride, int dtype,
                                   cudaStream_t st);
int b200_rope(void* q, void* k, const int64_t* positions, const float* cos_sin, int64_t T, int Hq, int Hk, int D,
              int rot_dim, int neox, int64_t max_pos, int64_t q_stride, int64_t k_stride, const int64_t* positions3,
              int sec0, int sec1, int interleaved, int dtype, cudaStream_t st);
int b200_reshape_and_cache(const void* k, const void* v, void* kv_cache, const int64_t* slots, int64_t T, int Hkv,
                           int D, int block_size, int64_t num_blocks, int64_t k_stride, int64_t v_stride, int dtype,
                           cudaStream_t st);
int b200_concat_and_cache_mla(const void* kv_c, const void* k_pe, void* cache, const int64_t* slots, int64_t T,
                              int rank, int rope, int64_t total_slots, int64_t kvc_stride, int64_t kpe_stride, int fp8,
                              int dtype, cudaStream_t st);
int b200_indexer_prep(const void* q, const void* k, const void* ln_w, const void* ln_b, const int64_t* positions,
                      const float* cos_sin, const void* head_w, float wscale, void* q_out, float* w_out, void* cache,
                      const int64_t* slots, int64_t T, int H, int64_t max_pos, int64_t total_slots, int64_t q_stride,
                      int64_t k_stride, int64_t hw_stride, float eps, int ue8m0, int64_t q_lo, int64_t q_hi, int block_size, int dtype,
                      cudaStream_t st);
int b200_indexer_k_quant_and_cache(const void* k, void* cache, const int64_t* slots, int64_t T, int64_t total_slots,
                                   int ue8m0, int64_t k_stride, int block_size, int dtype, cudaStream_t st);
int b200_convert_req_index(int32_t* out, const int32_t* req_id, const int32_t* block_table, const int32_t* idx,
                           int64_t T, int topk, int block_size, int max_blocks, int num_reqs, cudaStream_t st);
int b200_copy_blocks(void* cache, const int64_t* src, const int64_t* dst, int64_t n_pairs, int64_t bytes_per_block,
                     int64_t num_blocks, cudaStream_t st);
int b200_merge_attn_states(void* out, float* lse_out, const void* o1, const float* lse1, const void* o2,
                           const float* lse2, int64_t rows, int D, int dtype, cudaStream_t st);

// ---- attention ------------------------------------------------------------------------------
int b200_paged_attention(void* out, const void* q, const void* kv_cache, const int* block_tables, const int* seq_lens,
                         const int* qsl, const float* sinks, float* ws_o, float* ws_lse, int64_t T, int B, int Hq,
                         int Hkv, int D, int block_size, int max_blocks, int64_t num_blocks, int max_query_len,
                         int num_splits, int window, float scale, int decode_layout, int dtype, cudaStream_t st);

// Decode-shaped paged GQA attention on tcgen05 with TMA-fed KV tiles (attention/decode_umma.cu): head dim 128,
// at most 16 packed query rows per KV head, cache blocks of a multiple of 64 tokens.  `tmap`: the cache as a 2-D
// [blocks * 2 * Hkv * block_size, 128] tensor, 64 x 64 boxes, 128-byte swizzle.  Returns 3 for shapes it does not serve.
int b200_decode_attention_umma(void* out, const void* q, const void* tmap, const int* block_tables,
                               const int* seq_lens, const int* qsl, const float* sinks, float* ws_o, float* ws_lse,
                               int* status, int64_t T, int B, int Hq, int Hkv, int D, int block_size, int max_blocks,
                               int64_t num_blocks, int max_query_len, int num_splits, int window, float scale,
                               int early_meta, int dtype, cudaStream_t st);

// Dense paged MLA decode on tcgen05 (attention/mla_decode_umma.cu): cache blocks of 64 tokens, at most 32 query
// tokens per request.  `tmap`: the cache as a 2-D [blocks * 64, 576] 16-bit tensor, 64 x 64 boxes, 128-byte swizzle.
// early_meta as for b200_decode_attention_umma.  Returns 3 for shapes it does not serve.
int b200_mla_decode_umma(void* out, const void* q, const void* tmap, const int* block_tables, const int* seq_lens,
                         const int* qsl, float* ws_o, float* ws_lse, int* status, int64_t T, int B, int N,
                         int block_size, int max_blocks, int64_t num_blocks, int max_query_len, int num_splits,
                         float scale, int early_meta, int dtype, unsigned long long* trace, cudaStream_t st);

int b200_mla_decode_max_clusters(int R, int S, int dtype);
int b200_prefill_attention_umma(void* out, float* lse, const void* tmQ, const void* tmKV, const int* block_tables,
                                const int* seq_lens, const int* qsl, const float* sinks, int* status, int B, int Hq, int Hkv,
                                int D, int block_size, int max_blocks, int64_t num_blocks, int max_query_len, int window,
                                float scale, int dtype, unsigned long long* trace, cudaStream_t st);
int b200_mla_prefill_umma(void* out, float* lse, const void* tmQ, const void* tmKV, const void* tmKpe, const int* kv_starts,
                          const int* kv_lens, const int* qsl, int* status, int B, int Hq, int max_query_len, int causal,
                          float scale, int dtype, unsigned long long* trace, cudaStream_t st);
int b200_gather_mla_rows(void* out, const void* cache, const int32_t* slots, int64_t M, int64_t total_slots, int fp8,
                         int dtype, cudaStream_t st);
int b200_quant_int8_token(void* q, float* scale, const void* x, const float* static_scale, int64_t rows, int K,
                          int64_t x_stride, int dtype, cudaStream_t st);
int b200_indexer_logits_umma(float* logits, const void* tmQ, const float* w, const void* cache, const void* tmK,
                             const int* block_tables, const int* seq_lens, const int* qsl, int* status, int B,
                             int max_query_len, int max_blocks, int64_t num_blocks, int64_t ld, int64_t t_lo, int64_t t_hi,
                             cudaStream_t st);

int b200_merge_splits(void* out, const float* ws_o, const float* ws_lse, int64_t rows, int Hq, int D, int splits,
                      int64_t T, int dtype, cudaStream_t st);
// Absorbed MLA attention over the latent cache: dense paged (indices == null) or sparse by index list.
int b200_mla_attention(void* out, const void* q, const void* kv, const int* block_tables, const int* seq_lens,
                       const int* qsl, const int* req_of_token, const int* indices, float* ws_o, float* ws_lse,
                       int64_t T, int B, int N, int block_size, int max_blocks, int64_t total_slots, int topk,
                       int num_splits, float scale, int dtype, cudaStream_t st);

// Lightning indexer: fp8 scores over the paged key cache (per block: key rows, then scales), then per-row top-k (unordered, -1 padded)
int b200_indexer_logits(float* logits, const void* q_fp8, const float* w, const void* k_cache, const int* block_tables,
                        const int* seq_lens, const int* qsl, const int* req_of_token, int64_t T, int B, int block_size,
                        int max_blocks, int64_t total_slots, int64_t ld_logits, int64_t t0, cudaStream_t st);
int b200_topk_rows(int* out, const float* logits, const int* row_len, int64_t rows, int64_t ld, int k, int64_t max_len,
                   cudaStream_t st);

// ---- MoE / fp8 activation quantisation --------------------------------------------------------
int b200_moe_route(float* out_w, int* out_ids, const void* logits, const float* bias, int64_t T, int E, int k, int mode,
                   int renorm, int n_group, int topk_group, float scale, int64_t stride, int dtype, cudaStream_t st);
int b200_moe_permute(void* x_sorted, int* pos_of_pair, int* lod, int* counts, int* cursor, const void* x, const int* ids,
                     const int* emap, int64_t T, int k, int H, int E_local, int E_global, int64_t x_stride,
                     int64_t max_rows, int dtype, cudaStream_t st);
int b200_moe_unpermute(void* out, const void* y_sorted, const int* pos_of_pair, const float* w, int64_t T, int k, int H,
                       int dtype, cudaStream_t st);
int b200_router_gemm_small(float* out, const void* x, int64_t x_stride, const void* w, const void* bias,
                           int64_t T_, int N, int K, int dtype, cudaStream_t st);
int b200_router_route_small(float* out_w, int* out_ids, const void* x, int64_t x_stride, const void* w,
                            const void* wbias, const float* bias, int64_t T_, int E, int K, int k, int mode,
                            int renorm, int n_group, int topk_group, float scale, int dtype, cudaStream_t st);
int b200_moe_small_pairs();
int b200_moe_prepare_small(void* x_sorted, float* scale_t, int64_t s_stride, int* pos_of_pair, int* lod,
                           const void* x, const int* ids, const int* emap, int64_t T_, int k, int H, int E_local,
                           int E_global, int64_t x_stride, int quant, int dtype, cudaStream_t st);
int b200_act_mul_quant_fp8(void* q, float* scale_t, const void* h, int64_t rows, int I, int64_t s_stride, int act,
                           const int* rows_valid_ptr, int dtype, cudaStream_t st);
int b200_quant_fp8_group(void* q, float* scale_t, const void* x, int64_t rows, int K, int64_t x_stride, int64_t s_stride,
                         int ue8m0, const int* rows_valid_ptr, int dtype, cudaStream_t st);

// ---- communication over NVLink peer memory ----------------------------------------------------
int b200_allreduce_max_ctas();
int64_t b200_allreduce_flag_bytes();
int b200_oneshot_allreduce(void* const* bufs, const void* in, void* out, void* residual, const void* weight,
                           uint32_t* epochs, int* status, int64_t parity_bytes, int64_t flags_offset, int rank,
                           int nranks, int rows, int H, float eps, int gemma, int grid, uint32_t spin_limit, int dtype,
                           cudaStream_t st);

int b200_ll_allreduce(void* const* bufs, const void* in, void* out, void* residual, const void* weight,
                      uint32_t* epochs, int* status, int64_t slot_bytes, int rank, int nranks, int rows, int H,
                      float eps, int gemma, int grid, uint32_t spin_limit, int skip_push, int dtype, cudaStream_t st);

// Reduce-scatter consumer: sum R partial rows + residual, RMSNorm, push the row to every rank (see rs_norm_ag.cu)
typedef struct RsNormArgs {
  const void* stage; const void* rs_flags;
  void* xfull[8]; void* ag_flags[8];
  void* reset_a; void* reset_b; int reset_a_n, reset_b_n;
  void* residual; const void* weight; int* status;
  int rank, R, Tloc, H, rs_bn, n_tiles, ag_bn, rows_per_cta, max_tt, gemma, dtype;
  float eps; unsigned spin_limit;
} RsNormArgs;
int b200_rs_norm_ag(const RsNormArgs* a, cudaStream_t st);
int b200_sp_wait(const void* flags, int n_tt, unsigned expect, unsigned spin_limit, int* status, cudaStream_t st);

// ---- sampling ---------------------------------------------------------------------------------
int b200_topk_topp_sample(int64_t* out, const void* logits, int64_t rows, int V, int64_t stride,
                          const float* temperature, const int* top_k, const float* top_p, const float* noise,
                          int64_t noise_stride, uint64_t seed, uint64_t step, int dtype, cudaStream_t st);
int b200_repetition_penalty(void* logits, int64_t rows, int V, int64_t stride, const int64_t* tokens,
                            int64_t tok_stride, int max_tokens, const int* n_tokens, const float* penalty,
                            uint32_t* seen, int dtype, cudaStream_t st);
int b200_rejection_sample(int64_t* out, int64_t B, int S, const int64_t* draft_ids, const int* cu_draft,
                          const float* target_probs, const float* draft_probs, int V, const int64_t* bonus,
                          const uint8_t* is_greedy, const float* uniform, const float* recover_q, uint64_t seed,
                          uint64_t step, cudaStream_t st);

// ---- gated delta net / conv / MTP glue --------------------------------------------------------
int b200_causal_conv1d_fwd(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* w,
                           const void* bias, const int* cu, int R, void* states, const int* slots,
                           const uint8_t* has_init, int C, int W, int act, int64_t T_, int dtype, cudaStream_t st);
int b200_causal_conv1d_update(void* out, int64_t out_stride, const void* x, int64_t x_stride, void* states,
                              const void* w, const void* bias, const int* slots, int64_t B, int C, int W, int act,
                              int dtype, cudaStream_t st);
int b200_gdn_gating(float* g, float* beta, const void* a, int64_t a_stride, const void* b, int64_t b_stride,
                    const float* A_log, const float* dt_bias, int H, int64_t T_, int dtype, cudaStream_t st);
int b200_gdn_recurrent(void* out, int64_t o_stride, const void* q, const void* k, int64_t qk_stride, const void* v,
                       int64_t v_stride, const float* g, const float* beta, float* states, const int* cu,
                       const int* slots, const uint8_t* has_init, int R, int Hk, int Hv, int Dk, int Dv, float scale,
                       int l2norm, int dtype, cudaStream_t st);
int b200_sigmoid_gate_mul(void* out, const void* o, const void* gate, int64_t gate_stride, int D, int64_t T_,
                          int dtype, cudaStream_t st);
int b200_mtp_concat_norm(void* out, const void* embed, const void* hidden, const void* we, const void* wh,
                         const int64_t* pos, int64_t T_, int H, float eps, int dtype, cudaStream_t st);

// ---- LoRA ---------------------------------------------------------------------------------------
int b200_lora_shrink(float* out, const void* x, int64_t x_stride, const void* A, const int* ids, int64_t T_, int r,
                     int K, float scale, int dtype, cudaStream_t st);
int b200_lora_expand(void* out, int64_t out_stride, int offset, const float* h, const void* B, const int* ids,
                     int64_t T_, int N, int r, int add, int dtype, cudaStream_t st);

// ---- expert-parallel dispatch / combine over peer memory (see comm/ep_a2a.cu) --------------------
typedef struct EpArgs {
  void* peer[8];             // every rank's symmetric buffer (index = rank)
  int64_t off_x, off_scale, off_ids, off_w, off_recv_flag, off_comb, off_comb_flag;
  const void* x;             // local payload rows [T][x_row_bytes] (bf16, or fp8 already quantised)
  const float* x_scale_t;    // fp8 payload: transposed scales [H/128][scale_stride], else null
  int64_t x_row_bytes, scale_stride;
  const int* topk_ids;       // [T][k] global expert ids
  const float* topk_w;       // [T][k]
  int* send_count;           // [R] zero between calls
  int* sent_slot;            // [T][R]
  int* recv_count;           // [R]
  int* prev_count;           // [R]
  int* ticket;               // [3] zero between calls
  uint32_t* epoch;           // [1]
  int* status;
  int64_t T;
  int rank, R, cap, H, k, E, row_bytes;
  unsigned spin_limit;
} EpArgs;
int b200_ep_dispatch(const EpArgs* a, cudaStream_t st);
int b200_ep_permute_scales(float* scale_t, int64_t s_stride, const float* recv_scale, const int* pos_of_pair,
                           int64_t pairs, int k, int ngroups, cudaStream_t st);
int b200_ep_combine(const EpArgs* a, const void* y_sorted, const int* pos_of_pair, void* out, const void* addend,
                    int dtype, cudaStream_t st);

#ifdef __cplusplus
}
#endif
