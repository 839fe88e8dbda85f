"""Dense GQA decoders: Llama / Qwen2 / Qwen3 / InternLM2 / Seed-OSS / Mistral shapes.

In the reference these run on upstream model files and the plugin only contributes OOT layers, the
attention backend and the communicator (``vllm_kunlun/models/__init__.py:24-31``); ``seed_oss.py``
and ``internlm2.py`` are plain dense decoders on the plugin's ``Attention``.  One decode-step call
chain (``v1/attention/backends/kunlun_attn.py:751-949``): add+RMSNorm -> qkv GEMM -> (q/k norm) ->
RoPE -> cache write -> attention -> o_proj (all-reduce) -> add+RMSNorm -> gate_up -> SiLU*up -> down.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..parallel.state import get_state
from .layers import (DTYPES, ColumnParallelLinear, ParallelLMHead, RMSNorm, RowParallelLinear,
                     VocabParallelEmbedding, get_cos_sin_cache, param, reduce_add_rmsnorm, sp_sync, UnquantizedLinearMethod)


ACT_FUSION = [os.environ.get("B200_FUSE_ACT", "1") != "0"]  # also switched off while LoRA adapters wrap gate / up


class GQAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        st = get_state()
        tp = st.tp_size
        self.layer_idx = layer_idx
        self.cfg = cfg
        self.head_dim = cfg.head_dim
        self.v_head_dim = cfg.v_head_dim
        assert cfg.num_heads % tp == 0
        self.num_heads = cfg.num_heads // tp
        self.kv_replicated = tp > cfg.num_kv_heads
        self.num_kv_heads = max(1, cfg.num_kv_heads // tp)
        kv_total = cfg.num_kv_heads * cfg.head_dim
        v_total = cfg.num_kv_heads * cfg.v_head_dim
        if self.kv_replicated:
            # each rank keeps one KV head; the checkpoint slice is chosen at load time
            sizes = [cfg.q_size, self.head_dim, self.v_head_dim]
            repl = [False, True, True]
        else:
            sizes, repl = [cfg.q_size, kv_total, v_total], [False, False, False]
        quant = cfg.quantization if cfg.attn_quantization == "same" else cfg.attn_quantization
        self.qkv_proj = ColumnParallelLinear(cfg.hidden_size, sizes, bias=cfg.qkv_bias, dtype=dtype,
                                             device=device, quant=quant, replicate=repl)
        # the all-reduce of o_proj is fused into the add+RMSNorm that follows (reduce_add_rmsnorm)
        self.o_proj = RowParallelLinear(cfg.num_heads * cfg.v_head_dim, cfg.hidden_size, bias=cfg.o_bias,
                                        dtype=dtype, device=device, quant=quant, reduce_results=False)
        self.q_norm = self.k_norm = None
        if cfg.qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        self.scale = cfg.head_dim ** -0.5
        self.window = cfg.sliding_window if cfg.layer_is_sliding(layer_idx) else None
        self.sinks = param(self.num_heads, dtype=torch.float32, device=device) if cfg.attention_sinks else None
        self.cos_sin = get_cos_sin_cache(cfg.rotary_dim, cfg.max_position, cfg.rope_theta, cfg.rope_scaling, device)

    def kv_head_for_rank(self, part: int) -> int:
        """Row offset in the checkpoint K (part 1) / V (part 2) tensor for a replicated KV head."""
        st = get_state()
        head = st.tp_rank * self.cfg.num_kv_heads // st.tp_size
        return head * (self.head_dim if part == 1 else self.v_head_dim)

    def forward(self, hidden):
        ctx = get_forward_context()
        md = ctx.attn
        kv_cache = ctx.kv_caches[self.layer_idx]
        if self.v_head_dim != self.head_dim:
            raise NotImplementedError("asymmetric V head dim goes through models.mimo")
        proj = self.qkv_proj
        if (hidden.is_cuda and type(proj) is ColumnParallelLinear and type(proj.method) is UnquantizedLinearMethod
                and isinstance(kv_cache, torch.Tensor) and "forward" not in proj.__dict__):  # not wrapped (LoRA)
            from ..ops import gemm_cuda
            if gemm_cuda.qkv_epilogue_ok(hidden, proj.weight, self.head_dim, self.cfg.rotary_dim, kv_cache):
                # decode-sized batch: the projection's epilogue splits, normalises, rotates and writes the cache
                q = gemm_cuda.gemm_decode_qkv(
                    hidden, proj.weight, proj.bias, md.positions, self.cos_sin,
                    None if self.q_norm is None else self.q_norm.weight,
                    None if self.k_norm is None else self.k_norm.weight,
                    self.cfg.rms_norm_eps, self.num_heads, self.num_kv_heads, self.cfg.rope_neox, self.cfg.gemma_norm,
                    kv_cache, md.slot_mapping)
                return self._attend(q, kv_cache, md)
        qkv = proj(hidden)
        q = ops.qkv_split_norm_rope_cache(
            qkv, md.positions, self.cos_sin,
            None if self.q_norm is None else self.q_norm.weight,
            None if self.k_norm is None else self.k_norm.weight,
            self.cfg.rms_norm_eps, self.num_heads, self.num_kv_heads, self.head_dim, self.cfg.rope_neox,
            kv_cache, md.slot_mapping, self.cfg.gemma_norm)
        return self._attend(q, kv_cache, md)

    def _attend(self, q, kv_cache, md):
        T = q.shape[0]
        o = ops.paged_attention(
            q.view(T, self.num_heads, self.head_dim), kv_cache, md.block_tables, md.seq_lens,
            md.query_start_loc, self.scale, md.max_query_len, md.max_seq_len, self.window, self.sinks,
            md.seq_lens_cpu, md.query_start_loc_cpu, workspace=md.workspace,
            num_decodes=md.num_decodes, decode_query_len=1 + md.num_spec_tokens,
            num_decode_tokens=md.num_decode_tokens,
            stable_metadata=True)  # the runner fills lengths / block tables by host copies before the step
        return self.o_proj(o.reshape(T, self.num_heads * self.head_dim))


class GatedMLP(nn.Module):
    def __init__(self, hidden, inter, dtype, device, quant=None, act="silu", bias=False, reduce_results=True,
                 tp_size=None, tp_rank=None):
        super().__init__()
        self.gate_up_proj = ColumnParallelLinear(hidden, [inter, inter], bias=bias, dtype=dtype, device=device,
                                                 quant=quant, tp_size=tp_size, tp_rank=tp_rank)
        self.down_proj = RowParallelLinear(inter, hidden, bias=bias, dtype=dtype, device=device, quant=quant,
                                           reduce_results=reduce_results, tp_size=tp_size, tp_rank=tp_rank)
        self.act = act
        self.act_fused = False  # gate_up weight rows interleaved for the fused activation epilogue

    def forward(self, x):
        if self.act_fused:
            gu = self.gate_up_proj
            return self.down_proj(ops.linear_gated_act(x, gu.weight, gu.bias, self.act))
        return self.down_proj(ops.act_and_mul(self.gate_up_proj(x), self.act))

    # The fused layout is an in-place row permutation of the loaded weight: checkpoints are loaded and saved in
    # the plain [gate | up] order.
    def set_act_fused(self, on: bool) -> None:
        from ..ops.gemm_cuda import interleave_gate_up
        gu = self.gate_up_proj
        w = getattr(gu, "weight", None)
        eligible = (type(gu.method).__name__ == "UnquantizedLinearMethod" and w is not None and w.is_cuda
                    and w.dtype in (torch.bfloat16, torch.float16) and (w.shape[0] // 2) % 64 == 0
                    and self.act in ("silu", "gelu_tanh") and ACT_FUSION[0])
        if on == self.act_fused or (on and not eligible):
            return
        w.data.copy_(interleave_gate_up(w.data, inverse=not on))
        if gu.bias is not None:
            gu.bias.data.copy_(interleave_gate_up(gu.bias.data, inverse=not on))
        self.act_fused = on

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        from ..ops.gemm_cuda import interleave_gate_up
        sd = super().state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
        if self.act_fused:
            for name in ("weight", "bias"):
                key = f"{prefix}gate_up_proj.{name}"
                if key in sd and sd[key] is not None:
                    sd[key] = interleave_gate_up(sd[key], inverse=True)
        return sd


class DenseDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        self.self_attn = GQAAttention(cfg, layer_idx, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.gemma_norm)
        self.mlp = self.build_mlp(cfg, layer_idx, dtype, device)
        # both row-parallel outputs of a plain dense layer feed reduce_add_rmsnorm directly
        self.self_attn.o_proj.push_ok = True
        if type(self.mlp) is GatedMLP:
            self.mlp.down_proj.push_ok = True

    def build_mlp(self, cfg, layer_idx, dtype, device):
        return GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quantization,
                        cfg.hidden_act, cfg.mlp_bias, reduce_results=False)

    def forward(self, hidden, residual, partial: bool = False):
        """``hidden`` is a row-parallel partial sum when ``partial`` (previous layer's MLP output);
        the returned hidden is again a partial (tp > 1) to be reduced by the next norm."""
        hidden, residual = reduce_add_rmsnorm(hidden, residual, self.input_layernorm, partial)
        hidden = self.self_attn(hidden)
        hidden, residual = reduce_add_rmsnorm(hidden, residual, self.post_attention_layernorm, True)
        hidden = self.mlp(hidden)
        return hidden, residual


# checkpoint name fragment -> (fused param fragment, shard id)
STACKED = [
    (".q_proj.", ".qkv_proj.", 0), (".k_proj.", ".qkv_proj.", 1), (".v_proj.", ".qkv_proj.", 2),
    (".gate_proj.", ".gate_up_proj.", 0), (".up_proj.", ".gate_up_proj.", 1),
]


class DenseForCausalLM(nn.Module):
    """Pipeline-parallel aware causal LM (``SupportsPP`` pattern: each stage owns a layer slice and
    passes ``(hidden, residual)`` on, ``models/deepseek_v2.py:1102-1158``)."""

    layer_cls = DenseDecoderLayer
    post_layer_hook = None  # callable(layer_idx, hidden, residual): lets a wrapper touch the stream between layers
    aux_hidden_state_layers: tuple = ()  # EAGLE-3 target interface (``models/interfaces.py`` of the reference)
    aux_hidden = None

    def set_aux_hidden_state_layers(self, layers) -> None:
        self.aux_hidden_state_layers = tuple(layers)

    def get_eagle3_aux_hidden_state_layers(self) -> tuple:
        n = self.cfg.num_layers
        return (2, n // 2, n - 3) if n >= 6 else tuple(range(min(3, n)))

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype or DTYPES[cfg.dtype]
        self.device = torch.device(device)
        st = get_state()
        per = -(-cfg.num_layers // st.pp_size)
        self.first_layer = st.pp_rank * per
        self.last_layer = min(cfg.num_layers, self.first_layer + per)
        self.embed_tokens = (VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, self.dtype, device)
                             if st.is_first_pp or cfg.tie_word_embeddings else None)
        self.layers = nn.ModuleDict({
            str(i): self.layer_cls(cfg, i, self.dtype, device) for i in range(self.first_layer, self.last_layer)})
        self.norm = self.lm_head = None
        if st.is_last_pp:
            self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, self.dtype, device, cfg.gemma_norm)
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, self.dtype, device)
            if cfg.tie_word_embeddings and self.embed_tokens is not None:
                self.lm_head.weight = self.embed_tokens.weight

    # ---- forward ----
    def forward(self, input_ids, hidden=None, residual=None):
        if hidden is None:
            hidden = self.embed_tokens(input_ids)
        partial = False
        aux = []
        for i in range(self.first_layer, self.last_layer):
            if i in self.aux_hidden_state_layers:  # EAGLE-3: the stream entering layer i (needs a complete sum)
                aux += [self._complete(hidden, residual, partial)] * self.aux_hidden_state_layers.count(i)
            hidden, residual = self.layers[str(i)](hidden, residual, partial)
            partial = True
            if self.post_layer_hook is not None:
                self.post_layer_hook(i, hidden, residual)
        self.aux_hidden = torch.cat(aux, -1) if aux else None
        if self.norm is None:
            st = get_state()
            if st.tp_size > 1:  # hand a fully reduced activation to the next pipeline stage
                from .layers import SPPartial
                assert not isinstance(hidden, SPPartial), "sequence-parallel mode is not combined with PP"
                hidden = st.tp_comm.all_reduce(hidden)
            return hidden, residual
        hidden, _ = reduce_add_rmsnorm(hidden, residual, self.norm, partial)
        sp_sync()
        return hidden, None

    def _complete(self, hidden, residual, partial: bool):
        st = get_state()
        if partial and st.tp_size > 1:
            hidden = st.tp_comm.all_reduce(hidden.clone())
        return hidden if residual is None else hidden + residual

    def compute_logits(self, hidden):
        return self.lm_head.logits(hidden)

    # ---- KV cache ----
    def kv_cache_spec(self, block_size: int):
        """Per-layer ``(shape_per_block, dtype)`` for layers this stage owns."""
        st = get_state()
        kvh = max(1, self.cfg.num_kv_heads // st.tp_size)
        return {i: ((2, kvh, block_size, self.cfg.head_dim), self.dtype)
                for i in range(self.first_layer, self.last_layer)}

    # ---- weights ----
    def init_random(self, seed: int = 0, std: float = 0.02):
        """Seeded ``N(0, std)`` weights, norm weights = 1, biases/sinks ~ N(0, std)."""
        g = torch.Generator(device=self.device).manual_seed(seed + 1000 * get_state().tp_rank)
        g_rep = torch.Generator(device=self.device).manual_seed(seed + 7)  # replicated parameters: same on all ranks
        replicated = self.replicated_param_names()
        for name, p in self.named_parameters():
            if p.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                continue
            if name.endswith("layer_scalar"):
                p.data.fill_(1.0)
            elif name.endswith("norm.weight") or "layernorm.weight" in name:
                p.data.fill_(0.0 if self.cfg.gemma_norm else 1.0)
            else:
                gen = g_rep if name in replicated else g
                p.data.copy_((torch.randn(p.shape, generator=gen, device=self.device, dtype=torch.float32) * std)
                             .to(p.dtype))
        self.finish_loading()

    def replicated_param_names(self) -> set:
        from .layers import ReplicatedLinear
        out = set()
        for mname, m in self.named_modules():
            if isinstance(m, ReplicatedLinear):
                out.update(f"{mname}.{n}" for n, _ in m.named_parameters(recurse=False))
        return out

    def finish_loading(self):
        for m in self.modules():
            meth = getattr(m, "method", None)
            if meth is not None:
                meth.process_weights_after_loading(m)
            if isinstance(m, GatedMLP):
                m.set_act_fused(True)

    def _resolve(self, name: str):
        """Checkpoint tensor name -> (module, param name, shard id) or None when not on this stage."""
        name = name.removeprefix("model.")
        shard = None
        plain = name
        for ck, fused, sid in STACKED:
            if ck in name:
                name, shard = name.replace(ck, fused), sid
                break
        if shard is not None and self._walk(name.split(".")) is None and self._walk(plain.split(".")) is not None:
            # the module keeps this projection on its own (MLA without a low-rank query: ``self_attn.q_proj``)
            name, shard = plain, None
        parts = name.split(".")
        mod = self
        for i, p in enumerate(parts[:-1]):
            if p == "layers":
                continue
            if i > 0 and parts[i - 1] == "layers":
                if p not in self.layers:
                    return None
                mod = self.layers[p]
                continue
            if not hasattr(mod, p) or getattr(mod, p) is None:
                return None
            mod = getattr(mod, p)
        return mod, parts[-1], shard

    def _walk(self, parts):
        """The module that owns parameter path ``parts`` on this stage, or None."""
        mod = self
        for i, p in enumerate(parts[:-1]):
            if p == "layers":
                continue
            if i > 0 and parts[i - 1] == "layers":
                if p not in self.layers:
                    return None
                mod = self.layers[p]
                continue
            if not hasattr(mod, p) or getattr(mod, p) is None:
                return None
            mod = getattr(mod, p)
        return mod

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        loaded = set()
        for m in self.modules():
            if isinstance(m, GatedMLP):
                m.set_act_fused(False)  # checkpoints carry the plain [gate | up] order
        for name, w in weights:
            if "rotary_emb.inv_freq" in name:
                continue
            if name == "lm_head.weight" and self.cfg.tie_word_embeddings:
                continue
            r = self._resolve(name)
            if r is None:
                continue
            mod, pname, shard = r
            if shard is not None:
                shard += getattr(mod, "shard_offset", 0)
            if not hasattr(mod, pname) or getattr(mod, pname) is None:
                continue
            kw = {}
            attn = None
            if isinstance(mod, ColumnParallelLinear) and any(mod.replicate):
                attn = self._attn_owner(name)
                if attn is not None:
                    kw["kv_head_shard"] = attn.kv_head_for_rank
            if hasattr(mod, "load"):
                mod.load(pname, w, shard, **kw) if kw else mod.load(pname, w, shard)
            else:
                getattr(mod, pname).data.copy_(w)
            loaded.add(name)
        self.finish_loading()
        return loaded

    def _attn_owner(self, ckpt_name: str):
        parts = ckpt_name.removeprefix("model.").split(".")
        if len(parts) > 2 and parts[0] == "layers" and parts[1] in self.layers:
            return getattr(self.layers[parts[1]], "self_attn", None)
        return None
