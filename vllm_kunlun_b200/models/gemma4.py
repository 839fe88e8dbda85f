"""Gemma-family decoder: sandwich norms, (1 + w) RMSNorm, GELU-tanh gated MLP, per-layer sliding window,
scaled embeddings, q/k norm, final-logit soft-capping, cross-layer KV sharing, optional MoE blocks.

Reference: ``vllm_kunlun/models/gemma4.py`` (per-layer sliding window and cross-layer KV sharing :327-412, per-layer
inputs, MoE router) and ``ops/rotary_embedding/gemma4_rope.py:56-76`` (proportional RoPE: only a fraction of each
head is rotated, the rest passes through).  KV sharing: the last ``num_kv_shared_layers`` layers own no K/V
projection output in the cache; they attend over the cache written by the latest earlier layer of the same kind
(sliding / full).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..parallel.state import get_state
from .dense import GatedMLP, GQAAttention
from .layers import ReplicatedLinear, RMSNorm, VocabParallelEmbedding, param, reduce_add_rmsnorm
from .moe import FusedExperts, MoEForCausalLM


def kv_source_layer(cfg: ModelConfig, i: int) -> int:
    """Layer whose KV cache layer ``i`` reads (itself unless it is a KV-shared layer)."""
    first_shared = cfg.num_layers - cfg.num_kv_shared_layers
    if cfg.num_kv_shared_layers <= 0 or i < first_shared:
        return i
    kind = cfg.layer_is_sliding(i)
    for j in range(first_shared - 1, -1, -1):
        if cfg.layer_is_sliding(j) == kind:
            return j
    return i


def layer_attention_config(cfg: ModelConfig, i: int) -> ModelConfig:
    """The configuration as layer ``i``'s attention sees it: Gemma-4 full-attention layers may have their own head
    size and, when their values are their keys, their own KV head count."""
    if cfg.layer_is_sliding(i) or not (cfg.global_head_dim or cfg.attention_k_eq_v):
        return cfg
    import dataclasses
    hd = cfg.global_head_dim or cfg.head_dim
    kvh = cfg.num_global_kv_heads if (cfg.attention_k_eq_v and cfg.num_global_kv_heads) else cfg.num_kv_heads
    return dataclasses.replace(cfg, head_dim=hd, v_head_dim=hd, rotary_dim=hd, num_kv_heads=kvh)


class Gemma4Attention(GQAAttention):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        cfg = layer_attention_config(cfg, layer_idx)
        super().__init__(cfg, layer_idx, dtype, device)
        self.k_eq_v = cfg.attention_k_eq_v and not cfg.layer_is_sliding(layer_idx)
        self.kv_layer = kv_source_layer(cfg, layer_idx)
        if cfg.attn_scale is not None:
            self.scale = cfg.attn_scale
        kind = "sliding" if cfg.layer_is_sliding(layer_idx) else "full"
        if kind in cfg.rope_per_type:       # rotary parameters of this layer's type
            from .layers import get_cos_sin_cache
            theta, scaling = cfg.rope_per_type[kind]
            self.cos_sin = get_cos_sin_cache(self.head_dim, cfg.max_position, theta, scaling, device)

    def forward(self, hidden):
        if self.kv_layer == self.layer_idx:
            if not self.cfg.v_norm:
                return super().forward(hidden)
            # V is RMS-normalised per head (no weight) before it goes to the cache
            ctx = get_forward_context()
            md, cfg = ctx.attn, self.cfg
            kv_cache = ctx.kv_caches[self.layer_idx]
            qkv = self.qkv_proj(hidden)
            T = qkv.shape[0]
            v0 = (self.num_heads + self.num_kv_heads) * self.head_dim
            v = qkv[:, v0:].reshape(T * self.num_kv_heads, self.head_dim).float()
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)
            qkv = torch.cat([qkv[:, :v0], v.to(qkv.dtype).view(T, -1)], -1)
            q = ops.qkv_split_norm_rope_cache(
                qkv, md.positions, self.cos_sin, None if self.q_norm is None else self.q_norm.weight,
                None if self.k_norm is None else self.k_norm.weight, cfg.rms_norm_eps, self.num_heads, self.num_kv_heads,
                self.head_dim, cfg.rope_neox, kv_cache, md.slot_mapping, cfg.gemma_norm)
            return self._attend(q, kv_cache, md)
        # KV-shared layer: only the query is used; keys / values come from the source layer's cache
        ctx = get_forward_context()
        md, cfg = ctx.attn, self.cfg
        qkv = self.qkv_proj(hidden)
        T = qkv.shape[0]
        q = ops.qkv_split_norm_rope_cache(
            qkv, md.positions, self.cos_sin, None if self.q_norm is None else self.q_norm.weight,
            None if self.k_norm is None else self.k_norm.weight, cfg.rms_norm_eps, self.num_heads, self.num_kv_heads,
            self.head_dim, cfg.rope_neox, None, md.slot_mapping, cfg.gemma_norm)
        o = ops.paged_attention(
            q.view(T, self.num_heads, self.head_dim), ctx.kv_caches[self.kv_layer], md.block_tables, md.seq_lens,
            md.query_start_loc, self.scale, md.max_query_len, md.max_seq_len, self.window, self.sinks, md.seq_lens_cpu,
            md.query_start_loc_cpu, workspace=md.workspace, num_decodes=md.num_decodes,
            decode_query_len=1 + md.num_spec_tokens, num_decode_tokens=md.num_decode_tokens)
        return self.o_proj(o.reshape(T, self.num_heads * self.head_dim))


class Gemma4Router(nn.Module):
    """RMS-normalise (no weight), multiply by a learned per-channel scale and ``hidden ** -0.5``, project to expert
    scores; softmax over ALL experts, keep the top k, renormalise them to sum 1, then multiply each by its expert's
    learned scale."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.scale = param(cfg.hidden_size, dtype=dtype, device=device)
        self.proj = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, dtype=dtype, device=device)
        self.per_expert_scale = param(cfg.num_experts, dtype=dtype, device=device)

    def forward(self, x):
        cfg = self.cfg
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)
        xf = (xf * self.scale.float() * cfg.hidden_size ** -0.5).to(x.dtype)
        w, ids = ops.moe_route(ops.router_gemm(xf, self.proj.weight, None), cfg.num_experts_per_tok, "softmax", True,
                               None, 1, 1, 1.0)
        return w * self.per_expert_scale.float()[ids.long()], ids


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        def norm():
            return RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        self.input_layernorm, self.post_attention_layernorm = norm(), norm()
        self.pre_feedforward_layernorm, self.post_feedforward_layernorm = norm(), norm()
        self.self_attn = Gemma4Attention(cfg, layer_idx, dtype, device)
        shared = cfg.num_kv_shared_layers > 0 and layer_idx >= cfg.num_layers - cfg.num_kv_shared_layers
        inter = cfg.intermediate_size * (2 if cfg.double_wide_mlp and shared else 1)
        self.mlp = GatedMLP(cfg.hidden_size, inter, dtype, device, cfg.quantization, cfg.hidden_act,
                            cfg.mlp_bias, reduce_results=False)
        # sparse block BESIDE the dense MLP (reference gemma4.py:131-252,520-535,612-630): the router reads the
        # stream before the MLP; both branches are normed on their own, added, and normed once more
        self.moe = cfg.layer_is_moe(layer_idx)
        if self.moe:
            self.router = Gemma4Router(cfg, dtype, device)
            self.experts = FusedExperts(cfg, dtype, device)
            self.post_feedforward_layernorm_1, self.post_feedforward_layernorm_2 = norm(), norm()
            self.pre_feedforward_layernorm_2 = norm()
        # per-layer inputs (reference gemma4.py:553-581,632-640): a gate from the stream selects from this layer's
        # slice of the per-token embedding, which is projected back, normed and added; then the layer scalar
        self.ple = cfg.per_layer_input_size
        if self.ple:
            self.per_layer_input_gate = ReplicatedLinear(cfg.hidden_size, self.ple, dtype=dtype, device=device)
            self.per_layer_projection = ReplicatedLinear(self.ple, cfg.hidden_size, dtype=dtype, device=device)
            self.post_per_layer_input_norm = norm()
        if self.ple or cfg.layer_scalar:
            self.layer_scalar = param(1, dtype=dtype, device=device)

    def add_per_layer_input(self, m, residual, per_layer_input):
        """``per_layer_input [T, ple]``: returns the complete stream (no residual left over)."""
        h = m + residual
        gate = torch.nn.functional.gelu(self.per_layer_input_gate(h).float(), approximate="tanh").to(h.dtype)
        h = h + self.post_per_layer_input_norm(self.per_layer_projection(gate * per_layer_input))
        return h * self.layer_scalar

    def forward(self, hidden, residual, partial: bool = False):
        """``hidden`` is the complete (already reduced and post-normed) output of the previous layer."""
        if residual is None:
            residual = hidden
            h = self.input_layernorm(hidden)
        else:
            h, residual = self.input_layernorm(hidden, residual)
        a = self.self_attn(h)
        a, _ = reduce_add_rmsnorm(a, None, self.post_attention_layernorm, True)
        h, residual = self.pre_feedforward_layernorm(a, residual)
        m = self.mlp(h)
        if self.moe:
            m, _ = reduce_add_rmsnorm(m, None, self.post_feedforward_layernorm_1, True)
            w, ids = self.router(residual)
            e = self.experts(self.pre_feedforward_layernorm_2(residual), w, ids)
            e, _ = reduce_add_rmsnorm(e, None, self.post_feedforward_layernorm_2, True)
            return self.post_feedforward_layernorm(m + e), residual
        m, _ = reduce_add_rmsnorm(m, None, self.post_feedforward_layernorm, True)
        return m, residual


class Gemma4ForCausalLM(MoEForCausalLM):
    layer_cls = Gemma4DecoderLayer

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=None):
        super().__init__(cfg, device, dtype)
        # sqrt(hidden) rounded to the model's dtype, as a device scalar (creating it inside forward would be a
        # host-to-device copy, which a CUDA-graph capture does not allow)
        self.register_buffer("embed_scale", torch.tensor(cfg.hidden_size ** 0.5, dtype=self.dtype, device=device),
                             persistent=False)
        self.ple = cfg.per_layer_input_size
        if self.ple:
            assert get_state().pp_size == 1, "per-layer inputs are computed from the embeddings on the first stage"
            L = cfg.num_layers
            self.embed_tokens_per_layer = VocabParallelEmbedding(cfg.per_layer_vocab_size or cfg.vocab_size, L * self.ple,
                                                                 self.dtype, device)
            self.per_layer_model_projection = ReplicatedLinear(cfg.hidden_size, L * self.ple, dtype=self.dtype,
                                                               device=device)
            self.per_layer_projection_norm = RMSNorm(self.ple, cfg.rms_norm_eps, self.dtype, device, cfg.gemma_norm)

    def per_layer_inputs(self, input_ids, embeds):
        """``[T, L, ple]``: (norm(proj(embeds) / sqrt(hidden)) + per-layer token embedding * sqrt(ple)) / sqrt(2);
        tokens outside the per-layer vocabulary (multimodal placeholders) look up row 0 (reference
        ``gemma4.py:725-775``)."""
        L, P = self.cfg.num_layers, self.ple
        V = self.cfg.per_layer_vocab_size or self.cfg.vocab_size
        ids = torch.where((input_ids >= 0) & (input_ids < V), input_ids, torch.zeros_like(input_ids))
        tok = self.embed_tokens_per_layer(ids).view(-1, L, P) * (P ** 0.5)
        proj = (self.per_layer_model_projection(embeds) * (self.cfg.hidden_size ** -0.5)).view(-1, L, P)
        proj = self.per_layer_projection_norm(proj.reshape(-1, P)).view(-1, L, P)
        return (proj + tok.to(proj.dtype)) * (2.0 ** -0.5)

    def forward(self, input_ids, hidden=None, residual=None):
        if hidden is None:
            hidden = self.embed_tokens(input_ids)
            hidden = hidden * self.embed_scale
            hook = getattr(self, "input_embeds_hook", None)
            ple_ids = input_ids
            if hook is not None:  # multimodal wrapper: image rows replace the placeholder embeddings
                hidden, rows = hook(hidden)
                if rows is not None and self.ple:
                    # the per-layer token embedding of a placeholder row is the padding token's; the projected part
                    # is computed from the soft token itself
                    ple_ids = input_ids.index_fill(0, rows, int((self.cfg.vision or {}).get("pad_token_id", 0)))
        else:
            ple_ids = input_ids
        ple = self.per_layer_inputs(ple_ids, hidden) if self.ple else None
        for i in range(self.first_layer, self.last_layer):
            layer = self.layers[str(i)]
            hidden, residual = layer(hidden, residual)
            if ple is not None:
                hidden, residual = layer.add_per_layer_input(hidden, residual, ple[:, i].contiguous()), None
            elif self.cfg.layer_scalar:
                hidden, residual = (hidden + residual) * layer.layer_scalar, None
        if self.norm is None:
            return hidden, residual
        if residual is None:
            return self.norm(hidden), None
        hidden, _ = self.norm(hidden, residual)  # layer outputs are complete: no reduction here
        return hidden, None

    def compute_logits(self, hidden):
        lg = super().compute_logits(hidden)
        cap = self.cfg.final_logit_softcapping
        if cap:
            lg = (torch.tanh(lg.float() / cap) * cap).to(lg.dtype)
        return lg

    def kv_cache_spec(self, block_size: int):
        st = get_state()
        spec = {}
        for i in range(self.first_layer, self.last_layer):
            if kv_source_layer(self.cfg, i) != i:
                continue
            lc = layer_attention_config(self.cfg, i)
            spec[i] = ((2, max(1, lc.num_kv_heads // st.tp_size), block_size, lc.head_dim), self.dtype)
        return spec

    def load_weights(self, weights):
        # full-attention layers whose values are their keys have no v_proj tensor: the fused projection's V rows
        # take the K weight (V = k_proj(x), before the key's norm and rotation)
        out, loaded = [], set()
        for name, w in weights:
            if ".experts." in name and w.dim() == 3:
                # layers.L.experts.{gate_up_proj [E, 2 I, H] (gate rows first), down_proj [E, H, I]}; the multimodal
                # checkpoints spell it layers.L.moe.experts.*
                parts = name.removeprefix("model.").split(".")
                layer = self.layers[parts[1]] if parts[1] in self.layers else None
                if layer is not None and getattr(layer, "moe", False):
                    for e in range(w.shape[0]):
                        if parts[-1] == "down_proj":
                            layer.experts.load_expert(e, "down_proj", "weight", w[e])
                        else:
                            half = w.shape[1] // 2
                            layer.experts.load_expert(e, "gate_proj", "weight", w[e, :half])
                            layer.experts.load_expert(e, "up_proj", "weight", w[e, half:])
                    loaded.add(name)
                continue
            out.append((name, w))
            if self.cfg.attention_k_eq_v and ".self_attn.k_proj." in name:
                parts = name.removeprefix("model.").split(".")
                if parts[0] == "layers" and parts[1].isdigit() and not self.cfg.layer_is_sliding(int(parts[1])):
                    out.append((name.replace(".k_proj.", ".v_proj."), w))
        return loaded | super().load_weights(out)
