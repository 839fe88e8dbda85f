"""Dispatcher ops (``torch.ops.b200.*``) over the kernels, for hosts that trace models instead of calling Python.

The engine of this package calls ``ops.*`` directly.  A host that captures graphs by tracing (vLLM's compiled
mode, ``torch.export``) needs ops the dispatcher knows: a schema, declared mutations, and a fake implementation for
shape propagation.  The reference wraps its vendor kernels the same way - 54 ``torch.library.custom_op`` definitions
in ``vllm_kunlun/ops/_custom_ops.py`` (norms :255-555, ``split_norm_rope_neox`` :577, activations :699-759, MoE
routing / sort / grouped GEMM / un-permute :781-1413, int8 / int4 GEMMs :1045, :1416-1535, :1707-1883, cache writes
:1588, quantisers :1633, :1912, indexer logits :1994-2145, sparse MLA :2148-2335, top-k :2399, LoRA :2435-2880) -
and declares ``mutates_args=()`` on all of them, including the ones that write an argument.  Here every op that
writes an argument is exposed in mutating form (trailing underscore, returns nothing, mutation declared), the
others in functional form; twelve names of the reference that are empty stubs there (fp8 quantisers, fused norm +
quant) have real implementations here where this package has the kernel.

One table, ``OPS``: name -> (function, mutated argument names, fake implementation).
"""
from typing import List, Optional, Tuple

import torch

from .. import ops
from ..schema import direct_register_custom_op

_done = False
Tensor = torch.Tensor


def _copy_back(dst, src):
    if src is not dst and src.data_ptr() != dst.data_ptr():
        dst.copy_(src)


# ----------------------------------------------------------------------------- norms / activations
def rms_norm(x: Tensor, weight: Tensor, eps: float, gemma: bool = False) -> Tensor:
    return ops.rmsnorm(x, weight, eps, gemma)


def fused_add_rms_norm_(x: Tensor, residual: Tensor, weight: Tensor, eps: float, gemma: bool = False) -> None:
    """``residual += x; x = norm(residual) * weight``, both in place (``_C::add_rmsnorm`` / ``gemma_add_rmsnorm``)."""
    out, res = ops.add_rmsnorm(x, residual, weight, eps, gemma)
    _copy_back(x, out)
    _copy_back(residual, res)


def rms_norm_gated(x: Tensor, z: Tensor, weight: Tensor, eps: float, norm_before_gate: bool = True) -> Tensor:
    return ops.rms_norm_gated(x, z, weight, eps, norm_before_gate)


def l2norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    return ops.l2norm(x, eps)


def act_and_mul(x: Tensor, act: str = "silu") -> Tensor:
    """``silu`` / ``gelu_tanh`` / ``swigluoai`` gated activations (``_C::silu_and_mul``, ``_C::swigluoai_and_mul``)."""
    return ops.act_and_mul(x, act)


def quick_gelu(x: Tensor) -> Tensor:
    return ops.quick_gelu(x)


# ----------------------------------------------------------------------------- rotary / caches
def rotary_embedding_(q: Tensor, k: Tensor, positions: Tensor, cos_sin_cache: Tensor, head_dim: int,
                      neox: bool = True) -> None:
    q2, k2 = ops.rope(q, k, positions, cos_sin_cache, head_dim, neox)
    _copy_back(q, q2)
    _copy_back(k, k2)


def mrotary_embedding_(q: Tensor, k: Tensor, positions3: Tensor, cos_sin_cache: Tensor, head_dim: int,
                       sections: List[int], interleaved: bool = False) -> None:
    q2, k2 = ops.mrope(q, k, positions3, cos_sin_cache, head_dim, sections, interleaved)
    _copy_back(q, q2)
    _copy_back(k, k2)


def split_norm_rope_cache_(qkv: Tensor, positions: Tensor, cos_sin_cache: Tensor, q_weight: Optional[Tensor],
                           k_weight: Optional[Tensor], eps: float, num_heads: int, num_kv_heads: int, head_dim: int,
                           neox: bool, kv_cache: Tensor, slot_mapping: Tensor, q_out: Tensor,
                           gemma: bool = False) -> None:
    """Fused qkv split + per-head q/k RMSNorm + RoPE + paged-cache write (``_C::split_norm_rope_neox`` followed by
    ``reshape_and_cache_flash`` in the reference); the rotated queries land in ``q_out``."""
    q = ops.qkv_split_norm_rope_cache(qkv, positions, cos_sin_cache, q_weight, k_weight, eps, num_heads, num_kv_heads,
                                      head_dim, neox, kv_cache, slot_mapping, gemma)
    q_out.copy_(q.reshape(q_out.shape))


def reshape_and_cache_(k: Tensor, v: Tensor, kv_cache: Tensor, slot_mapping: Tensor) -> None:
    ops.reshape_and_cache(k, v, kv_cache, slot_mapping)


def concat_and_cache_mla_(kv_c: Tensor, k_pe: Tensor, kv_cache: Tensor, slot_mapping: Tensor) -> None:
    ops.concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping)


def indexer_k_quant_and_cache_(k: Tensor, k_cache: Tensor, slot_mapping: Tensor, ue8m0: bool = True) -> None:
    ops.indexer_k_quant_and_cache(k, k_cache, slot_mapping, ue8m0)


def convert_req_index_to_global_index(req_id: Tensor, block_table: Tensor, token_indices: Tensor,
                                      block_size: int) -> Tensor:
    return ops.convert_req_index_to_global_index(req_id, block_table, token_indices, block_size)


# ----------------------------------------------------------------------------- attention
def paged_attention_(out: Tensor, q: Tensor, kv_cache: Tensor, block_tables: Tensor, seq_lens: Tensor,
                     query_start_loc: Tensor, scale: float, max_query_len: int, max_seq_len: int, window: int = 0,
                     sinks: Optional[Tensor] = None, num_decodes: int = 0, decode_query_len: int = 1) -> None:
    """Unified varlen paged GQA attention (the graph-splitting op ``vllm::unified_attention_with_output_kunlun``)."""
    o = ops.paged_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, max_query_len, max_seq_len,
                            window or None, sinks, out=out if out.is_cuda else None, num_decodes=num_decodes,
                            decode_query_len=decode_query_len, num_decode_tokens=num_decodes * decode_query_len)
    _copy_back(out, o)


def merge_attn_states(o1: Tensor, lse1: Tensor, o2: Tensor, lse2: Tensor) -> Tuple[Tensor, Tensor]:
    return ops.merge_attn_states(o1, lse1, o2, lse2)


def mla_attention(q: Tensor, kv_cache: Tensor, block_tables: Tensor, seq_lens: Tensor, query_start_loc: Tensor,
                  scale: float, kv_lora_rank: int, max_query_len: int, max_seq_len: int) -> Tensor:
    return ops.mla_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, kv_lora_rank, max_query_len,
                             max_seq_len)


def sparse_mla_attention(q: Tensor, kv_cache: Tensor, indices: Tensor, scale: float, d_v: int = 512) -> Tensor:
    """``_C::sparse_prefill_fwd_opt`` / ``_C::fwd_kvcache_mla`` of the reference in one op."""
    return ops.sparse_mla_attention(q, kv_cache, indices, scale, d_v)


def indexer_topk(q_fp8: Tensor, q_scale: Tensor, weights: Tensor, k_cache: Tensor, block_tables: Tensor,
                 seq_lens: Tensor, query_start_loc: Tensor, topk: int) -> Tensor:
    """``_C::I8_(paged_)mqa_logits`` + ``_C::fast_topkv2`` of the reference in one op."""
    return ops.indexer_topk(q_fp8, q_scale, weights, k_cache, block_tables, seq_lens, query_start_loc, topk)


# ----------------------------------------------------------------------------- GEMMs / quantisation
def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    return ops.linear(x, weight, bias)


def linear_gated_act(x: Tensor, weight_interleaved: Tensor, bias_interleaved: Optional[Tensor] = None,
                     act: str = "silu") -> Tensor:
    return ops.linear_gated_act(x, weight_interleaved, bias_interleaved, act)


def quant_fp8_per_group(x: Tensor, group: int = 128, ue8m0: bool = False) -> Tuple[Tensor, Tensor]:
    """``_C::dynamic_per_token_scaled_fp8_quant`` family (empty stubs in the reference)."""
    q, s = ops.quant_fp8_per_group(x, group, ue8m0)
    return q, s


def fp8_linear(x: Tensor, w_fp8: Tensor, w_scale_inv: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    return ops.fp8_linear(x, w_fp8, w_scale_inv, bias)


def int8_linear(x: Tensor, w_q: Tensor, w_scale: Tensor, bias: Optional[Tensor] = None,
                input_scale: Optional[Tensor] = None) -> Tensor:
    """W8A8 linear (``_C::cutlass_scaled_mm`` / ``_C::matmul`` of the reference)."""
    return ops.int8_linear(x, w_q, w_scale, bias, input_scale)


def bmm_heads(x: Tensor, w: Tensor) -> Tensor:
    return ops.bmm_heads(x, w)


# ----------------------------------------------------------------------------- MoE
def moe_route(logits: Tensor, k: int, scoring: str = "softmax", renormalize: bool = True,
              bias: Optional[Tensor] = None, n_group: int = 1, topk_group: int = 1,
              scale: float = 1.0) -> Tuple[Tensor, Tensor]:
    """``_C::moe_softmax_topk(_norm)`` / ``_C::moe_sigmoid_group_topk_norm`` / GPT-OSS routing."""
    w, ids = ops.moe_route(logits, k, scoring, renormalize, bias, n_group, topk_group, scale)[:2]
    return w, ids


def fused_moe(x: Tensor, w13: Tensor, w2: Tensor, topk_weights: Tensor, topk_ids: Tensor, act: str = "silu",
              b13: Optional[Tensor] = None, b2: Optional[Tensor] = None, w13_scale: Optional[Tensor] = None,
              w2_scale: Optional[Tensor] = None, expert_map: Optional[Tensor] = None) -> Tensor:
    """Permute -> grouped GEMM -> activation -> grouped GEMM -> weighted un-permute (``_C::moe_ffn_block`` /
    ``moe_pre_sorted`` + ``moe_fc`` + ``moe_post``); ``expert_map`` restricts the work to this rank's experts."""
    return ops.fused_moe(x, w13, w2, topk_weights, topk_ids, act, b13, b2, w13_scale, w2_scale, (128, 128), expert_map)


# ----------------------------------------------------------------------------- sampling
def argmax(logits: Tensor) -> Tensor:
    return ops.argmax(logits)


def topk_topp_sample(logits: Tensor, temperature: Optional[Tensor] = None, top_k: Optional[Tensor] = None,
                     top_p: Optional[Tensor] = None, noise: Optional[Tensor] = None, seed: int = 0) -> Tensor:
    return ops.topk_topp_sample(logits, temperature, top_k, top_p, noise, seed)


def apply_repetition_penalties_(logits: Tensor, token_ids: Tensor, num_tokens: Tensor, penalties: Tensor) -> None:
    _copy_back(logits, ops.apply_repetition_penalty(logits, token_ids, num_tokens, penalties))


# ----------------------------------------------------------------------------- linear attention
def causal_conv1d_update_(x: Tensor, conv_states: Tensor, weight: Tensor, bias: Optional[Tensor],
                          state_indices: Tensor, out: Tensor, activation: bool = True) -> None:
    out.copy_(ops.causal_conv1d_update(x, conv_states, weight, bias, state_indices, activation))


def fused_gdn_gating(A_log: Tensor, a: Tensor, b: Tensor, dt_bias: Tensor) -> Tuple[Tensor, Tensor]:
    g, beta = ops.fused_gdn_gating(A_log, a, b, dt_bias)
    return g, beta


# ----------------------------------------------------------------------------- LoRA
def lora_shrink(x: Tensor, lora_a: Tensor, token_lora_ids: Tensor, scale: float = 1.0) -> Tensor:
    """Per-token shrink (``_C::bgmv_shrink_lora`` / ``sgmv_shrink_lora``)."""
    return ops.lora_shrink(x, lora_a, token_lora_ids, scale)


def lora_expand_(h: Tensor, lora_b: Tensor, token_lora_ids: Tensor, out: Tensor, offset: int = 0,
                 add: bool = True) -> None:
    """Per-token expand into a column slice (``_C::bgmv_expand(_slice)_lora`` / ``sgmv_expand(_slice)_lora``)."""
    _copy_back(out, ops.lora_expand(h, lora_b, token_lora_ids, out, offset, add))


# ----------------------------------------------------------------------------- fake implementations
def _like(i=0):
    return lambda *a, **k: torch.empty_like(a[i])


def _none(*a, **k):
    return None


def _half_cols(x, *a, **k):
    return x.new_empty(*x.shape[:-1], x.shape[-1] // 2)


def _rows_of_weight(x, w, *a, **k):
    return x.new_empty(*x.shape[:-1], w.shape[0])


def _f_route(logits, k, *a, **kw):
    return (logits.new_empty(logits.shape[0], k, dtype=torch.float32),
            logits.new_empty(logits.shape[0], k, dtype=torch.int32))


def _f_quant(x, group=128, ue8m0=False):
    return (x.new_empty(x.shape, dtype=torch.float8_e4m3fn),
            x.new_empty(*x.shape[:-1], x.shape[-1] // group, dtype=torch.float32))


OPS = {
    "rms_norm": (rms_norm, (), _like()),
    "fused_add_rms_norm_": (fused_add_rms_norm_, ("x", "residual"), _none),
    "rms_norm_gated": (rms_norm_gated, (), _like()),
    "l2norm": (l2norm, (), _like()),
    "act_and_mul": (act_and_mul, (), _half_cols),
    "quick_gelu": (quick_gelu, (), _like()),
    "rotary_embedding_": (rotary_embedding_, ("q", "k"), _none),
    "mrotary_embedding_": (mrotary_embedding_, ("q", "k"), _none),
    "split_norm_rope_cache_": (split_norm_rope_cache_, ("kv_cache", "q_out"), _none),
    "reshape_and_cache_": (reshape_and_cache_, ("kv_cache",), _none),
    "concat_and_cache_mla_": (concat_and_cache_mla_, ("kv_cache",), _none),
    "indexer_k_quant_and_cache_": (indexer_k_quant_and_cache_, ("k_cache",), _none),
    "convert_req_index_to_global_index": (convert_req_index_to_global_index, (),
                                          lambda r, b, t, bs: t.new_empty(t.shape, dtype=torch.int32)),
    "paged_attention_": (paged_attention_, ("out",), _none),
    "merge_attn_states": (merge_attn_states, (), lambda o1, l1, o2, l2: (torch.empty_like(o1), torch.empty_like(l1))),
    "mla_attention": (mla_attention, (),
                      lambda q, kv, bt, sl, ql, scale, r, mq, ms: q.new_empty(q.shape[0], q.shape[1], r)),
    "sparse_mla_attention": (sparse_mla_attention, (),
                             lambda q, kv, idx, scale, d_v=512: q.new_empty(q.shape[0], q.shape[1], d_v)),
    "indexer_topk": (indexer_topk, (),
                     lambda q, qs, w, kc, bt, sl, ql, topk: q.new_empty(q.shape[0], topk, dtype=torch.int32)),
    "linear": (linear, (), _rows_of_weight),
    "linear_gated_act": (linear_gated_act, (), lambda x, w, b=None, act="silu": x.new_empty(*x.shape[:-1], w.shape[0] // 2)),
    "quant_fp8_per_group": (quant_fp8_per_group, (), _f_quant),
    "fp8_linear": (fp8_linear, (), lambda x, w, s, b=None: x.new_empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16)),
    "int8_linear": (int8_linear, (),
                    lambda x, w, s, b=None, i=None: x.new_empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16)),
    "bmm_heads": (bmm_heads, (), lambda x, w: x.new_empty(x.shape[0], x.shape[1], w.shape[2])),
    "moe_route": (moe_route, (), _f_route),
    "fused_moe": (fused_moe, (), _like()),
    "argmax": (argmax, (), lambda lg: lg.new_empty(lg.shape[0], dtype=torch.int64)),
    "topk_topp_sample": (topk_topp_sample, (), lambda lg, *a, **k: lg.new_empty(lg.shape[0], dtype=torch.int64)),
    "apply_repetition_penalties_": (apply_repetition_penalties_, ("logits",), _none),
    "causal_conv1d_update_": (causal_conv1d_update_, ("conv_states", "out"), _none),
    "fused_gdn_gating": (fused_gdn_gating, (),
                         lambda A, a, b, dt: (a.new_empty(a.shape, dtype=torch.float32), torch.empty_like(b))),
    "lora_shrink": (lora_shrink, (), lambda x, a, ids, scale=1.0: x.new_empty(x.shape[0], a.shape[1], dtype=torch.float32)),
    "lora_expand_": (lora_expand_, ("out",), _none),
}


def register_custom_ops() -> None:
    """Define the ``b200`` namespace once per process (``vllm.general_plugins`` entry point ``b200_ops``)."""
    global _done
    if _done:
        return
    _done = True
    for name, (fn, mutates, fake) in OPS.items():
        direct_register_custom_op(name, fn, list(mutates), fake_impl=fake)
