"""Qwen3-Next / Qwen3.5: hybrid decoder with Gated DeltaNet (linear attention) layers, gated full
attention every n-th layer, and a sparse-MoE block with a sigmoid-gated shared expert.

Reference: ``vllm_kunlun/models/qwen3_next.py`` - sparse MoE block with shared-expert gate (:142-259),
Gated DeltaNet layer (:262-781: conv1d fn / update, ``fused_gdn_gating``, chunked vs recurrent delta rule,
state write-back), gated attention with fused split + q/k norm + RoPE (:784-922), custom op
``vllm::gdn_attention_core`` (:1415-1450); metadata builder ``v1/attention/backends/gdn_attn.py:163-436``.

Layout choices here (differ from the checkpoint, converted at load time):
* ``in_proj`` output rows are ``[q | k | v | z]`` and ``in_proj_ba`` rows ``[b | a]`` (the checkpoint interleaves
  them per key head), so the conv input ``[q | k | v]`` is a contiguous column slice and TP shards whole heads.
* per-request state lives in two caches indexed by the request's state slot:
  ``conv [slots, W-1, C_local]`` and ``ssm [slots, Hv_local, Dv, Dk]`` (fp32).
* one varlen kernel serves prefill chunks and decode tokens alike (sequential scan with the state in
  registers), so mixed batches need no prefill/decode split.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..parallel.state import get_state
from .dense import GatedMLP, GQAAttention
from .layers import ColumnParallelLinear, RMSNorm, RowParallelLinear, param, reduce_add_rmsnorm
from .moe import MoEForCausalLM, SparseMoEBlock


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        st = get_state()
        tp = st.tp_size
        self.cfg, self.layer_idx = cfg, layer_idx
        assert cfg.gdn_num_k_heads % tp == 0 and cfg.gdn_num_v_heads % tp == 0
        self.hk, self.hv = cfg.gdn_num_k_heads // tp, cfg.gdn_num_v_heads // tp
        self.dk, self.dv = cfg.gdn_head_k_dim, cfg.gdn_head_v_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        kd, vd = cfg.gdn_num_k_heads * self.dk, cfg.gdn_num_v_heads * self.dv
        self.in_proj = ColumnParallelLinear(cfg.hidden_size, [kd, kd, vd, vd], dtype=dtype, device=device,
                                            quant=cfg.quantization)
        self.in_proj_ba = ColumnParallelLinear(cfg.hidden_size, [cfg.gdn_num_v_heads, cfg.gdn_num_v_heads], dtype=dtype,
                                               device=device)
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_weight = param(self.conv_dim, cfg.gdn_conv_kernel, dtype=dtype, device=device)
        self.A_log = param(self.hv, dtype=torch.float32, device=device)
        self.dt_bias = param(self.hv, dtype=torch.float32, device=device)
        self.norm = RMSNorm(self.dv, cfg.rms_norm_eps, dtype, device)
        self.out_proj = RowParallelLinear(vd, cfg.hidden_size, dtype=dtype, device=device, quant=cfg.quantization,
                                          reduce_results=False)

    def state_spec(self, dtype):
        return [((self.cfg.gdn_conv_kernel - 1, self.conv_dim), dtype), ((self.hv, self.dv, self.dk), torch.float32)]

    def forward(self, hidden):
        ctx = get_forward_context()
        md = ctx.attn
        conv_state, ssm_state = ctx.kv_caches[self.layer_idx]
        T = hidden.shape[0]
        qkvz = self.in_proj(hidden)
        ba = self.in_proj_ba(hidden)
        mixed = qkvz[:, : self.conv_dim]
        z = qkvz[:, self.conv_dim:]
        if md.max_query_len == 1:
            mixed = ops.causal_conv1d_update(mixed, conv_state, self.conv_weight, None, md.state_indices, True)
        else:
            mixed = ops.causal_conv1d_fn(mixed, self.conv_weight, None, md.query_start_loc, conv_state, md.state_indices,
                                         md.has_initial_state, True)
        g, beta = ops.fused_gdn_gating(self.A_log, ba[:, self.hv:], ba[:, : self.hv], self.dt_bias)
        q = mixed[:, : self.key_dim].view(T, self.hk, self.dk)
        k = mixed[:, self.key_dim:2 * self.key_dim].view(T, self.hk, self.dk)
        v = mixed[:, 2 * self.key_dim:].view(T, self.hv, self.dv)
        o = ops.gated_delta_rule(q, k, v, g, beta, ssm_state, md.query_start_loc, md.state_indices, md.has_initial_state,
                                 self.dk ** -0.5, True, md.query_start_loc_cpu)
        o = ops.rms_norm_gated(o.reshape(T * self.hv, self.dv), z.reshape(T * self.hv, self.dv), self.norm.weight,
                               self.cfg.rms_norm_eps, True)
        return self.out_proj(o.reshape(T, self.value_dim))

    # ---- checkpoint conversion: per-key-head interleaved rows -> [q | k | v | z] / [b | a]
    def load_qkvz(self, w: torch.Tensor, pname: str = "weight"):
        cfg = self.cfg
        Hk, rep = cfg.gdn_num_k_heads, cfg.gdn_num_v_heads // cfg.gdn_num_k_heads
        per = 2 * self.dk + 2 * rep * self.dv
        g = w.reshape(Hk, per, -1)
        q, k = g[:, : self.dk], g[:, self.dk:2 * self.dk]
        v = g[:, 2 * self.dk:2 * self.dk + rep * self.dv]
        z = g[:, 2 * self.dk + rep * self.dv:]
        for i, part in enumerate((q, k, v, z)):
            self.in_proj.load(pname, part.reshape(-1, w.shape[-1]), i)

    def load_ba(self, w: torch.Tensor):
        cfg = self.cfg
        Hk, rep = cfg.gdn_num_k_heads, cfg.gdn_num_v_heads // cfg.gdn_num_k_heads
        g = w.reshape(Hk, 2 * rep, -1)
        self.in_proj_ba.load("weight", g[:, :rep].reshape(-1, w.shape[-1]), 0)
        self.in_proj_ba.load("weight", g[:, rep:].reshape(-1, w.shape[-1]), 1)

    def load_conv(self, w: torch.Tensor):
        """Checkpoint ``conv1d.weight [C_total, 1, W]`` with channels ``[q | k | v]`` over all heads."""
        st = get_state()
        cfg = self.cfg
        w = w.reshape(w.shape[0], -1)
        kd, vd = cfg.gdn_num_k_heads * self.dk, cfg.gdn_num_v_heads * self.dv
        parts = [(0, kd, self.key_dim), (kd, kd, self.key_dim), (2 * kd, vd, self.value_dim)]
        dst = 0
        for off, _, loc in parts:
            self.conv_weight.data[dst:dst + loc].copy_(w[off + st.tp_rank * loc: off + (st.tp_rank + 1) * loc])
            dst += loc

    def load_head_vector(self, name: str, w: torch.Tensor):
        st = get_state()
        getattr(self, name).data.copy_(w[st.tp_rank * self.hv:(st.tp_rank + 1) * self.hv].float())


class GatedAttention(GQAAttention):
    """Full attention whose output is multiplied by ``sigmoid(gate)``; the gate is the second half of an
    enlarged q projection.  Fused row layout here: ``[gate | q | k | v]``."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__(cfg, layer_idx, dtype, device)
        st = get_state()
        kv_total = cfg.num_kv_heads * cfg.head_dim
        if self.kv_replicated:
            sizes, repl = [cfg.q_size, cfg.q_size, self.head_dim, self.head_dim], [False, False, True, True]
        else:
            sizes, repl = [cfg.q_size, cfg.q_size, kv_total, kv_total], [False] * 4
        self.qkv_proj = ColumnParallelLinear(cfg.hidden_size, sizes, bias=cfg.qkv_bias, dtype=dtype, device=device,
                                             quant=cfg.quantization, replicate=repl)
        self.qkv_proj.shard_offset = 1  # checkpoint k / v are partitions 2 / 3 of the fused row
        self.q_local = cfg.q_size // st.tp_size

    def kv_head_for_rank(self, part: int) -> int:
        return super().kv_head_for_rank(part - 1)

    def forward(self, hidden):
        ctx = get_forward_context()
        md = ctx.attn
        fused = self.qkv_proj(hidden)
        gate = fused[:, : self.q_local]
        kv_cache = ctx.kv_caches[self.layer_idx]
        pos3 = ctx.extras.get("mrope_positions") if ctx.extras else None
        if pos3 is not None:
            # Qwen3.5 with images in this step: three-axis rotary positions over the rotated part of each head
            cfg, T = self.cfg, fused.shape[0]
            qs, ks = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
            q = fused[:, self.q_local:self.q_local + qs].contiguous()
            k = fused[:, self.q_local + qs:self.q_local + qs + ks].contiguous()
            v = fused[:, self.q_local + qs + ks:].contiguous()
            if self.q_norm is not None:
                q = self.q_norm(q.view(-1, self.head_dim)).view(T, qs)
                k = self.k_norm(k.view(-1, self.head_dim)).view(T, ks)
            q, k = ops.mrope(q, k, pos3, self.cos_sin, self.head_dim, list(cfg.mrope_section), cfg.mrope_interleaved)
            ops.reshape_and_cache(k.view(T, self.num_kv_heads, self.head_dim), v.view(T, self.num_kv_heads, self.head_dim),
                                  kv_cache, md.slot_mapping)
        else:
            q = self._split_norm_rope_cache(fused, md, kv_cache)
        T = q.shape[0]
        o = ops.paged_attention(
            q.view(T, self.num_heads, self.head_dim), kv_cache, md.block_tables, md.seq_lens, md.query_start_loc,
            self.scale, md.max_query_len, md.max_seq_len, self.window, self.sinks, md.seq_lens_cpu,
            md.query_start_loc_cpu, workspace=md.workspace, num_decodes=md.num_decodes,
            decode_query_len=1 + md.num_spec_tokens, num_decode_tokens=md.num_decode_tokens)
        o = ops.sigmoid_gate_mul(o.reshape(T, self.q_local), gate)
        return self.o_proj(o)

    def _split_norm_rope_cache(self, fused, md, kv_cache):
        return ops.qkv_split_norm_rope_cache(
            fused[:, self.q_local:], md.positions, self.cos_sin,
            None if self.q_norm is None else self.q_norm.weight, None if self.k_norm is None else self.k_norm.weight,
            self.cfg.rms_norm_eps, self.num_heads, self.num_kv_heads, self.head_dim, self.cfg.rope_neox,
            kv_cache, md.slot_mapping, self.cfg.gemma_norm)

    def load_q_and_gate(self, w: torch.Tensor, pname: str = "weight"):
        """Checkpoint ``q_proj`` rows are ``[head][q(D) | gate(D)]``."""
        H, D = self.cfg.num_heads, self.head_dim
        g = w.reshape(H, 2, D, -1) if w.dim() == 2 else w.reshape(H, 2, D)
        tail = (w.shape[-1],) if w.dim() == 2 else ()
        self.qkv_proj.load(pname, g[:, 1].reshape(H * D, *tail), 0)
        self.qkv_proj.load(pname, g[:, 0].reshape(H * D, *tail), 1)


class Qwen3NextDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.is_linear = cfg.layer_is_linear_attn(layer_idx)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        if self.is_linear:
            self.linear_attn = GatedDeltaNet(cfg, layer_idx, dtype, device)
        else:
            self.self_attn = (GatedAttention if cfg.attn_output_gate else GQAAttention)(cfg, layer_idx, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        if cfg.layer_is_moe(layer_idx):
            self.mlp = SparseMoEBlock(cfg, dtype, device)
        else:
            self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quantization, cfg.hidden_act,
                                cfg.mlp_bias, reduce_results=False)

    def forward(self, hidden, residual, partial: bool = False):
        hidden, residual = reduce_add_rmsnorm(hidden, residual, self.input_layernorm, partial)
        hidden = self.linear_attn(hidden) if self.is_linear else self.self_attn(hidden)
        hidden, residual = reduce_add_rmsnorm(hidden, residual, self.post_attention_layernorm, True)
        return self.mlp(hidden), residual


class Qwen3NextForCausalLM(MoEForCausalLM):
    layer_cls = Qwen3NextDecoderLayer

    def kv_cache_spec(self, block_size: int):
        st = get_state()
        kvh = max(1, self.cfg.num_kv_heads // st.tp_size)
        return {i: ((2, kvh, block_size, self.cfg.head_dim), self.dtype)
                for i in range(self.first_layer, self.last_layer) if not self.cfg.layer_is_linear_attn(i)}

    def state_cache_spec(self):
        """Per-slot (not per-block) caches of the linear-attention layers."""
        return {i: self.layers[str(i)].linear_attn.state_spec(self.dtype)
                for i in range(self.first_layer, self.last_layer) if self.cfg.layer_is_linear_attn(i)}

    def init_random(self, seed: int = 0, std: float = 0.02):
        super().init_random(seed, std)
        for m in self.modules():
            if isinstance(m, GatedDeltaNet):
                m.A_log.data.uniform_(-1.0, 1.0)  # decay rates exp(-exp(A) * softplus(.)) well inside (0, 1)
                m.dt_bias.data.uniform_(-1.0, 1.0)
                m.conv_weight.data.mul_(10.0)  # keep the conv output away from zero under l2-norm

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        rest, loaded = [], set()
        for name, w in weights:
            if name.startswith("mtp."):
                continue
            n = name.removeprefix("model.").removeprefix("language_model.")
            parts = n.split(".")
            layer = self.layers[parts[1]] if len(parts) > 2 and parts[0] == "layers" and parts[1] in self.layers else None
            if layer is not None and parts[2] == "linear_attn":
                gdn = layer.linear_attn
                key = ".".join(parts[3:])
                if key.startswith("in_proj_qkvz."):
                    gdn.load_qkvz(w, parts[-1])
                elif key == "in_proj_ba.weight":
                    gdn.load_ba(w)
                elif key.startswith("in_proj_qkv."):
                    # Qwen3.5 keeps the projections apart and in plain order: [q | k | v] rows, then z, b and a
                    kd = self.cfg.gdn_num_k_heads * gdn.dk
                    for i, part in enumerate((w[:kd], w[kd:2 * kd], w[2 * kd:])):
                        gdn.in_proj.load(parts[-1], part, i)
                elif key.startswith("in_proj_z."):
                    gdn.in_proj.load(parts[-1], w, 3)
                elif key == "in_proj_b.weight":
                    gdn.in_proj_ba.load("weight", w, 0)
                elif key == "in_proj_a.weight":
                    gdn.in_proj_ba.load("weight", w, 1)
                elif key == "conv1d.weight":
                    gdn.load_conv(w)
                elif key in ("A_log", "dt_bias"):
                    gdn.load_head_vector(key, w)
                elif key == "norm.weight":
                    gdn.norm.weight.data.copy_(w)
                elif key.startswith("out_proj."):
                    gdn.out_proj.load(parts[-1], w)
                else:
                    continue
                loaded.add(name)
                continue
            if layer is not None and parts[2] == "self_attn" and parts[3] == "q_proj" and self.cfg.attn_output_gate:
                layer.self_attn.load_q_and_gate(w, parts[-1])
                loaded.add(name)
                continue
            if layer is not None and parts[2] == "mlp" and parts[3] == "shared_expert":
                name = name.replace(".shared_expert.", ".shared_experts.")
            rest.append((name, w))
        loaded |= super().load_weights(rest)
        return loaded

    @property
    def uses_state_cache(self) -> bool:
        return self.cfg.linear_attn_pattern > 0
