"""Attention backends: the ``AttentionBackend`` quadruple (impl / metadata / builder / KV-cache shape)
for paged GQA, MLA and sparse MLA.

Reference: ``KunlunAttentionBackend`` (``v1/attention/backends/kunlun_attn.py:59-125``), ``FlashMLABackend``
(``mla/flashmla.py:30-46``), ``FlashMLASparseBackend`` (``mla/flashmla_sparse.py:43-96``).  All backends here
support whole-step CUDA graphs for uniform decode batches (``q_len = 1 + num_spec``) because the kernels
read lengths, block tables and slot mappings from device memory."""
from __future__ import annotations

import torch

from .. import ops
from .metadata import AttentionMetadata


class MetadataBuilder:
    """Decode-first batch order; requests with ``q_len <= 1 + num_spec`` count as decodes."""

    cudagraph_support = "UNIFORM_BATCH"
    supports_update_block_table = True

    def __init__(self, num_spec_tokens: int = 0):
        self.reorder_batch_threshold = 1 + num_spec_tokens

    def reorder_batch(self, query_lens: list) -> list:
        thr = self.reorder_batch_threshold
        dec = [i for i, q in enumerate(query_lens) if q <= thr]
        pre = [i for i, q in enumerate(query_lens) if q > thr]
        return dec + pre

    def build(self, positions, slot_mapping, block_tables, seq_lens, query_start_loc, max_query_len, max_seq_len,
              num_decodes=0, num_decode_tokens=0, **kw) -> AttentionMetadata:
        B = seq_lens.shape[0]
        return AttentionMetadata(
            num_tokens=positions.shape[0], num_reqs=B, positions=positions, slot_mapping=slot_mapping,
            block_tables=block_tables, seq_lens=seq_lens, query_start_loc=query_start_loc,
            max_query_len=max_query_len, max_seq_len=max_seq_len, num_decodes=num_decodes,
            num_decode_tokens=num_decode_tokens, num_prefills=B - num_decodes, **kw)

    def build_for_cudagraph_capture(self, md: AttentionMetadata, max_model_len: int) -> AttentionMetadata:
        md.max_seq_len = max_model_len
        md.max_query_len = self.reorder_batch_threshold
        return md

    def build_for_drafting(self, md: AttentionMetadata) -> AttentionMetadata:
        return md  # the draft model runs on the target step's rows with the same metadata


class GQABackend:
    accept_output_buffer = True

    @staticmethod
    def get_name() -> str:
        return "B200_GQA"

    @staticmethod
    def get_supported_head_sizes():
        return [64, 128, 256]

    @staticmethod
    def get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size):
        return (num_blocks, 2, num_kv_heads, block_size, head_size)

    @staticmethod
    def get_metadata_cls():
        return AttentionMetadata

    @staticmethod
    def get_builder_cls():
        return MetadataBuilder

    @staticmethod
    def get_impl_cls():
        return GQAImpl


class GQAImpl:
    def __init__(self, num_heads, head_size, scale, num_kv_heads, sliding_window=None, sinks=None):
        self.num_heads, self.head_size, self.scale, self.num_kv_heads = num_heads, head_size, scale, num_kv_heads
        self.window, self.sinks = sliding_window, sinks

    def forward(self, q, k, v, kv_cache, md: AttentionMetadata, output=None):
        """``reshape_and_cache`` then unified paged attention (``kunlun_attn.py:751-949``)."""
        if md is None or md.is_dummy:  # profile run
            return output if output is not None else torch.zeros_like(q)
        T = q.shape[0]
        if k is not None:
            ops.reshape_and_cache(k.view(T, self.num_kv_heads, self.head_size),
                                  v.view(T, self.num_kv_heads, self.head_size), kv_cache, md.slot_mapping)
        return ops.paged_attention(q.view(T, self.num_heads, self.head_size), kv_cache, md.block_tables, md.seq_lens,
                                   md.query_start_loc, self.scale, md.max_query_len, md.max_seq_len, self.window,
                                   self.sinks, md.seq_lens_cpu, md.query_start_loc_cpu, out=output,
                                   workspace=md.workspace, num_decodes=md.num_decodes,
                                   decode_query_len=1 + md.num_spec_tokens, num_decode_tokens=md.num_decode_tokens)


class MLABackend(GQABackend):
    @staticmethod
    def get_name() -> str:
        return "B200_MLA"

    @staticmethod
    def get_supported_head_sizes():
        return [576]

    @staticmethod
    def get_kv_cache_shape(num_blocks, block_size, num_kv_heads=1, head_size=576):
        return (num_blocks, block_size, head_size)

    @staticmethod
    def get_impl_cls():
        return MLAImpl


class MLAImpl:
    can_return_lse_for_decode = False

    def __init__(self, num_heads, scale, kv_lora_rank=512):
        self.num_heads, self.scale, self.rank = num_heads, scale, kv_lora_rank

    def forward(self, q_absorbed, kv_c, k_pe, kv_cache, md: AttentionMetadata):
        if md is None or md.is_dummy:
            return torch.zeros(q_absorbed.shape[0], self.num_heads, self.rank, dtype=q_absorbed.dtype,
                               device=q_absorbed.device)
        if kv_c is not None:
            ops.concat_and_cache_mla(kv_c, k_pe, kv_cache, md.slot_mapping)
        return ops.mla_attention(q_absorbed, kv_cache, md.block_tables, md.seq_lens, md.query_start_loc, self.scale,
                                 self.rank, md.max_query_len, md.max_seq_len, md.seq_lens_cpu,
                                 md.query_start_loc_cpu, md.workspace)


class SparseMLABackend(MLABackend):
    @staticmethod
    def get_name() -> str:
        return "B200_MLA_SPARSE"

    @staticmethod
    def get_kv_cache_shape(num_blocks, block_size=64, num_kv_heads=1, head_size=576, cache_dtype="auto"):
        if cache_dtype == "fp8_ds_mla":
            return (num_blocks, block_size, 656)
        return (num_blocks, block_size, head_size)

    @staticmethod
    def get_impl_cls():
        return SparseMLAImpl


class SparseMLAImpl(MLAImpl):
    def __init__(self, num_heads, scale, kv_lora_rank=512, topk_tokens=2048):
        super().__init__(num_heads, scale, kv_lora_rank)
        self.topk = topk_tokens

    def forward(self, q_absorbed, kv_c, k_pe, kv_cache, md: AttentionMetadata, topk_local_indices=None):
        if md is None or md.is_dummy:
            return torch.zeros(q_absorbed.shape[0], self.num_heads, self.rank, dtype=q_absorbed.dtype,
                               device=q_absorbed.device)
        if kv_c is not None:
            ops.concat_and_cache_mla(kv_c, k_pe, kv_cache, md.slot_mapping)
        slots = ops.convert_req_index_to_global_index(md.req_id_per_token, md.block_tables, topk_local_indices,
                                                      kv_cache.shape[1])
        return ops.sparse_mla_attention(q_absorbed, kv_cache, slots, self.scale, self.rank)
