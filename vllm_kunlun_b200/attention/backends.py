"""Attention backends for upstream vLLM's V1 engine: ``AttentionBackend`` subclasses with their metadata
builders and implementations, selected by ``B200Platform.get_attn_backend_cls``.

Reference: ``KunlunAttentionBackend`` / builder / impl (``v1/attention/backends/kunlun_attn.py:59-125``,
``:447-693``, ``:696-949``), ``FlashMLABackend`` (``mla/flashmla.py:30-46``, ``:98-228``) and
``FlashMLASparseBackend`` (``mla/flashmla_sparse.py:43-96``, ``:749-813``).  The classes derive from the bases
of the installed vLLM and keep their constructor / ``build`` / ``forward`` signatures; the arithmetic runs in
this package's kernels (CUDA tensors) or its fp32 oracles (CPU tensors, used by the CPU tests).

Differences from the reference on purpose: the dense backend supports CUDA graphs for uniform decode batches
(``q_len = 1 + num_spec``) because the kernels read lengths, block tables and slot mappings from device memory;
the KV cache of one layer is ``[blocks, 2, kv_heads, block_size, head_size]`` (a page of one head contiguous,
which is what the TMA-fed decode kernel wants).

The standalone engine of this package does not go through these classes (its runner builds
:class:`vllm_kunlun_b200.attention.metadata.AttentionMetadata` directly)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

from .. import ops

try:
    from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionLayer,
                                           AttentionMetadataBuilder, AttentionType, CommonAttentionMetadata,
                                           MultipleOf)
    from vllm.v1.attention.backends.utils import split_decodes_and_prefills
    HAVE_VLLM = True
except Exception:  # pragma: no cover - vLLM is optional for the standalone engine
    HAVE_VLLM = False
    AttentionBackend = AttentionImpl = AttentionMetadataBuilder = object  # type: ignore
    AttentionLayer = CommonAttentionMetadata = object  # type: ignore


if HAVE_VLLM:

    @dataclass
    class GQAMetadata:
        """Per-step metadata of the dense paged backend (decode-first batch)."""
        num_actual_tokens: int
        max_query_len: int
        max_seq_len: int
        query_start_loc: torch.Tensor      # [B + 1] int32, device
        seq_lens: torch.Tensor             # [B] int32, device
        block_table: torch.Tensor          # [B, max_blocks] int32, device
        slot_mapping: torch.Tensor         # [T] int64, device
        num_decodes: int = 0
        num_decode_tokens: int = 0
        num_prefills: int = 0
        decode_query_len: int = 1
        causal: bool = True
        query_start_loc_cpu: Optional[torch.Tensor] = None
        seq_lens_cpu: Optional[torch.Tensor] = None
        workspace: Optional[object] = None

    class GQAMetadataBuilder(AttentionMetadataBuilder[GQAMetadata]):
        """Consumes upstream's ``CommonAttentionMetadata``.  Requests with at most ``1 + num_spec`` query tokens
        are pulled to the front of the batch (``reorder_batch_threshold``) and served by the decode kernel."""

        _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_BATCH
        supports_update_block_table: bool = True

        def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
            super().__init__(kv_cache_spec, layer_names, vllm_config, device)
            self._init_reorder_batch_threshold(1, supports_spec_as_decode=True)
            self.block_size = kv_cache_spec.block_size
            self.max_model_len = vllm_config.model_config.max_model_len
            self._workspace = None

        def _get_workspace(self, tokens: int, heads: int, head_size: int, device):
            if device.type != "cuda":
                return None
            from ..ops.attention_cuda import AttnWorkspace
            ws = self._workspace
            if ws is None or ws.max_tokens < tokens:
                ws = self._workspace = AttnWorkspace(max(tokens, 64), heads, head_size, 16, device)
            return ws

        def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
                  fast_build: bool = False) -> GQAMetadata:
            m = common_attn_metadata
            thr = self.reorder_batch_threshold or 1
            nd, npf, ndt, _ = split_decodes_and_prefills(m, decode_threshold=thr, require_uniform=True)
            spec = self.kv_cache_spec
            heads = getattr(spec, "num_kv_heads", 1)
            ws = None
            if nd:
                # query heads per rank are not part of the cache spec; size the split-KV scratch for the worst case
                # the model config allows on this rank
                par = self.vllm_config.parallel_config
                q_heads = self.vllm_config.model_config.get_num_attention_heads(par)
                ws = self._get_workspace(max(ndt, self.vllm_config.scheduler_config.max_num_seqs * thr), max(q_heads, heads),
                                         spec.head_size, m.seq_lens.device)
            return GQAMetadata(
                num_actual_tokens=m.num_actual_tokens, max_query_len=m.max_query_len, max_seq_len=m.max_seq_len,
                query_start_loc=m.query_start_loc, seq_lens=m.seq_lens, block_table=m.block_table_tensor,
                slot_mapping=m.slot_mapping, num_decodes=nd, num_decode_tokens=ndt, num_prefills=npf,
                decode_query_len=(ndt // nd) if nd else 1, causal=m.causal,
                query_start_loc_cpu=m.query_start_loc_cpu, seq_lens_cpu=getattr(m, "_seq_lens_cpu", None), workspace=ws)

        def build_for_cudagraph_capture(self, common_attn_metadata: CommonAttentionMetadata) -> GQAMetadata:
            md = self.build(0, common_attn_metadata)
            md.max_seq_len = self.max_model_len  # plan the split-KV grid for the longest context a replay may see
            return md

        def update_block_table(self, metadata: GQAMetadata, blk_table: torch.Tensor, slot_mapping: torch.Tensor):
            import copy
            md = copy.copy(metadata)
            md.block_table, md.slot_mapping = blk_table, slot_mapping
            return md

        def use_cascade_attention(self, *args, **kwargs) -> bool:
            return False

    class GQAImpl(AttentionImpl[GQAMetadata]):
        """Paged GQA attention: cache write, then decode rows on the tcgen05 decode kernel and prefill rows on the
        varlen kernel (the reference: ``reshape_and_cache_flash`` -> ``prefill_attention`` -> ``speculative_attention``,
        ``kunlun_attn.py:805-947``)."""

        def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                     alibi_slopes: Optional[list] = None, sliding_window: Optional[int] = None,
                     kv_cache_dtype: str = "auto", logits_soft_cap: Optional[float] = None,
                     attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name: Optional[str] = None,
                     sinks: Optional[torch.Tensor] = None) -> None:
            if alibi_slopes is not None:
                raise NotImplementedError("ALiBi is not implemented by the B200 attention kernels")
            if logits_soft_cap:
                raise NotImplementedError("logit soft-capping is not implemented by the B200 attention kernels")
            if attn_type != AttentionType.DECODER:
                raise NotImplementedError("only decoder self-attention is served by B200_GQA")
            if kv_cache_dtype not in ("auto", "bfloat16", "float16"):
                raise NotImplementedError(f"kv_cache_dtype={kv_cache_dtype!r}: the dense backend keeps a 16-bit cache")
            self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
            self.num_kv_heads = num_kv_heads or num_heads
            self.sliding_window = sliding_window
            self.kv_cache_dtype = kv_cache_dtype
            self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
            self.sinks = sinks

        def forward(self, layer: AttentionLayer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    kv_cache: torch.Tensor, attn_metadata: GQAMetadata, output: torch.Tensor,
                    output_scale: Optional[torch.Tensor] = None,
                    output_block_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
            assert output is not None, "the output buffer is provided by the attention layer"
            if output_scale is not None or output_block_scale is not None:
                raise NotImplementedError("fused output quantisation is not supported by B200_GQA")
            if attn_metadata is None:  # profiling run
                return output.fill_(0)
            md = attn_metadata
            T = md.num_actual_tokens
            H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_size
            q = query[:T].reshape(T, H, D)
            if key is not None and value is not None and self.kv_sharing_target_layer_name is None:
                ops.reshape_and_cache(key[:T].reshape(T, Hkv, D), value[:T].reshape(T, Hkv, D), kv_cache,
                                      md.slot_mapping[:T])
            out = output[:T].view(T, H, D) if output.is_contiguous() else None
            o = ops.paged_attention(
                q.contiguous(), kv_cache, md.block_table, md.seq_lens, md.query_start_loc, self.scale, md.max_query_len,
                md.max_seq_len, self.sliding_window, self.sinks, md.seq_lens_cpu, md.query_start_loc_cpu, out=out,
                workspace=md.workspace, num_decodes=md.num_decodes, decode_query_len=md.decode_query_len,
                num_decode_tokens=md.num_decode_tokens)
            if out is None or o.data_ptr() != out.data_ptr():
                output[:T].view(T, H, D).copy_(o)
            return output

    class GQABackend(AttentionBackend):
        accept_output_buffer: bool = True
        supported_dtypes: ClassVar[list] = [torch.float16, torch.bfloat16]
        supported_kv_cache_dtypes: ClassVar[list] = ["auto", "float16", "bfloat16"]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"  # the name upstream's registry gives to an out-of-tree backend (kunlun_attn.py:66-68)

        @staticmethod
        def get_impl_cls():
            return GQAImpl

        @staticmethod
        def get_builder_cls():
            return GQAMetadataBuilder

        @staticmethod
        def get_metadata_cls():
            return GQAMetadata

        @classmethod
        def get_supported_head_sizes(cls) -> list:
            return [64, 128, 256]

        @staticmethod
        def get_supported_kernel_block_sizes() -> list:
            return [MultipleOf(16)]

        @staticmethod
        def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                               cache_dtype_str: str = "auto") -> tuple:
            return (num_blocks, 2, num_kv_heads, block_size, head_size)

        @classmethod
        def supports_sink(cls) -> bool:
            return True

        @classmethod
        def supports_compute_capability(cls, capability) -> bool:
            return capability.major == 10

    # ------------------------------------------------------------------------------------------------ MLA
    from vllm.model_executor.layers.attention.mla_attention import (MLACommonBackend, MLACommonImpl, MLACommonMetadata,
                                                                    MLACommonMetadataBuilder)

    class MLAMetadataBuilder(MLACommonMetadataBuilder[MLACommonMetadata]):
        _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_BATCH

    class MLAImpl(MLACommonImpl[MLACommonMetadata]):
        """Weight-absorbed decode over the 576-wide latent cache on this package's MLA kernel; prefill, chunked
        context and the up-projections are upstream's common MLA code (``mla/common.py:1782-1843`` in the
        reference's fork)."""

        can_return_lse_for_decode: bool = False

        def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                     alibi_slopes: Optional[list], sliding_window: Optional[int], kv_cache_dtype: str,
                     logits_soft_cap: Optional[float], attn_type: str, kv_sharing_target_layer_name: Optional[str],
                     **mla_args) -> None:
            super().__init__(num_heads, head_size, scale, num_kv_heads, alibi_slopes, sliding_window, kv_cache_dtype,
                             logits_soft_cap, attn_type, kv_sharing_target_layer_name, **mla_args)
            if any([alibi_slopes, sliding_window, logits_soft_cap]):
                raise NotImplementedError("B200 MLA does not support alibi_slopes, sliding_window or logits_soft_cap")
            if attn_type != AttentionType.DECODER:
                raise NotImplementedError("only decoder self-attention is served by B200 MLA")

        def forward_mqa(self, q, kv_c_and_k_pe_cache: torch.Tensor, attn_metadata: MLACommonMetadata,
                        layer: AttentionLayer):
            assert kv_c_and_k_pe_cache.numel() > 0 and attn_metadata.decode is not None
            if type(q) is tuple:
                q = torch.cat(q, dim=-1)
            dec = attn_metadata.decode
            B = dec.seq_lens.shape[0]
            T = q.shape[0]
            q_len = max(1, T // max(B, 1))
            qsl = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32, device=q.device)
            o = ops.mla_attention(q.contiguous(), kv_c_and_k_pe_cache, dec.block_table, dec.seq_lens, qsl, self.scale,
                                  self.kv_lora_rank, max_query_len=q_len,
                                  max_seq_len=getattr(attn_metadata, "max_seq_len", 0) or 0)
            return o, None

    class MLABackend(MLACommonBackend):
        supported_kv_cache_dtypes: ClassVar[list] = ["auto", "bfloat16", "float16"]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return MLAImpl

        @staticmethod
        def get_builder_cls():
            return MLAMetadataBuilder

        @staticmethod
        def get_supported_kernel_block_sizes() -> list:
            return [64]

        @classmethod
        def get_supported_head_sizes(cls) -> list:
            return [576]

        @classmethod
        def supports_compute_capability(cls, capability) -> bool:
            return capability.major == 10

    class SparseMLABackend(MLABackend):
        """DeepSeek-V3.2 sparse MLA: cache ``(blocks, 64, 576)`` 16-bit or the 656-byte ``fp8_ds_mla`` rows
        (``flashmla_sparse.py:43-54,84-96``); attention over the top-k rows selected by the lightning indexer."""

        supported_kv_cache_dtypes: ClassVar[list] = ["auto", "bfloat16", "fp8_ds_mla"]

        @classmethod
        def is_sparse(cls) -> bool:
            return True

        @staticmethod
        def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                               cache_dtype_str: str = "auto") -> tuple:
            if cache_dtype_str == "fp8_ds_mla":
                return (num_blocks, block_size, 656)  # 512 fp8 + 4 fp32 scales + 64 16-bit rope dims per token
            return (num_blocks, block_size, head_size)

else:  # pragma: no cover
    GQABackend = MLABackend = SparseMLABackend = None  # type: ignore


def sparse_mla_forward(q: torch.Tensor, kv_cache: torch.Tensor, topk_indices: torch.Tensor, req_id_per_token,
                       block_table: torch.Tensor, scale: float, block_size: int = 64, d_v: int = 512) -> torch.Tensor:
    """Sparse MLA over request-local top-k indices: convert them to global cache slots
    (``convert_req_index_to_global_index``, ``flashmla_sparse.py:690-698``) and attend over the selected rows
    (``_forward_bf16_kv``, ``:631-720``)."""
    gidx = ops.convert_req_index_to_global_index(req_id_per_token, block_table, topk_indices, block_size)
    return ops.sparse_mla_attention(q, kv_cache, gidx, scale, d_v)
