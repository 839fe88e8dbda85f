"""Typed configuration objects and architecture presets.

The reference plugin receives its configuration from upstream vLLM
(``VllmConfig``) and only mutates it in
``vllm_kunlun/platforms/kunlun.py:147-245`` (block size 16 by default, 64 for
MLA / sparse MLA, eager fallbacks) and ``vllm_kunlun/models/config.py:619-643``
(per-architecture fix-ups).  This framework is standalone, so it owns the whole
configuration surface; the same fix-ups live in :meth:`EngineConfig.finalize`.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class RopeScaling:
    """YaRN parameters (``models/deepseek_v2.py:311-316,889-903`` in the reference)."""

    type: str = "none"  # "none" | "yarn" | "linear" | "llama3"
    factor: float = 1.0
    original_max_position: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    truncate: bool = True   # YaRN: round the correction range to whole dimensions (gpt-oss checkpoints say False)
    partial: float = 1.0    # "proportional": fraction of the head's angle pairs that rotate (the rest keep angle 0)


@dataclass
class ModelConfig:
    """Architecture description shared by every model family."""

    architecture: str = "LlamaForCausalLM"
    name: str = "unnamed"
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 11008
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    rope_neox: bool = True
    rotary_dim: Optional[int] = None
    max_position: int = 8192
    tie_word_embeddings: bool = False
    qkv_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    qk_norm: bool = False  # per-head q/k RMSNorm (Qwen3)
    hidden_act: str = "silu"  # "silu" | "swigluoai" | "gelu_tanh"
    gemma_norm: bool = False  # (1 + w) RMSNorm
    # sliding window / sinks (GPT-OSS, MiMo-V2, Gemma)
    sliding_window: Optional[int] = None
    sliding_window_pattern: int = 0  # every n-th layer is full attention; 0 = none sliding
    attention_sinks: bool = False
    v_head_dim: Optional[int] = None  # asymmetric V (MiMo-V2-Flash)
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    shared_expert_gate: bool = False  # Qwen2-MoE / Qwen3-Next sigmoid gate on the shared expert
    shared_intermediate_size: Optional[int] = None  # width of the shared expert when the checkpoint names it (else
    # num_shared_experts x moe_intermediate_size)
    first_dense_layers: int = 0
    moe_layer_freq: int = 1
    scoring_func: str = "softmax"  # "softmax" | "sigmoid"
    norm_topk_prob: bool = True
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    router_bias: bool = False  # e_score_correction_bias
    moe_bias: bool = False  # GPT-OSS experts carry biases
    # MLA
    use_mla: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    # DeepSeek-V3.2 lightning indexer
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    # MTP
    num_mtp_layers: int = 0
    # Gated DeltaNet (Qwen3-Next) hybrid
    linear_attn_pattern: int = 0  # every n-th layer is full attention, others GDN; 0 = none
    gdn_num_k_heads: int = 0
    gdn_num_v_heads: int = 0
    gdn_head_k_dim: int = 0
    gdn_head_v_dim: int = 0
    gdn_conv_kernel: int = 4
    # vision-language: tower description (depth, hidden, heads, patch, ...) and M-RoPE sections of the decoder
    vision: Optional[dict] = None
    mrope_section: tuple = ()
    mrope_interleaved: bool = False
    num_kv_shared_layers: int = 0  # Gemma: trailing layers that reuse an earlier layer's KV cache
    attn_scale: Optional[float] = None  # softmax scale override (Gemma query_pre_attn_scalar)
    final_logit_softcapping: float = 0.0
    # Gemma per-layer inputs ("PLE"): width of the per-layer embedding and the vocabulary it is looked up in
    per_layer_input_size: int = 0
    per_layer_vocab_size: int = 0
    layer_types: tuple = ()  # explicit "sliding_attention" / "full_attention" per layer (else sliding_window_pattern)
    rope_per_type: dict = field(default_factory=dict)  # layer type -> (theta, RopeScaling) when the types differ
    v_norm: bool = False  # RMS-normalise V per head, without a weight (Gemma-4)
    layer_scalar: bool = False  # a learned scalar multiplies the stream at the end of every layer (Gemma-4)
    double_wide_mlp: bool = False  # KV-shared layers have an MLP of twice the width (Gemma-4)
    global_head_dim: Optional[int] = None  # head size of the full-attention layers when it differs (Gemma-4)
    num_global_kv_heads: Optional[int] = None  # their KV head count when values are the keys (attention_k_eq_v)
    attention_k_eq_v: bool = False  # full-attention layers have no v_proj: V is the (un-normalised, un-rotated) K
    attn_output_gate: bool = False  # q_proj carries a sigmoid output gate (Qwen3-Next full-attention layers)
    # quantization of the checkpoint
    quantization: Optional[str] = None  # None | "fp8" | "int8" | "awq" | "gptq" | "w4a16"
    quantization_kw: dict = field(default_factory=dict)  # constructor arguments of the linear method (group size, bits, ...)
    attn_quantization: Optional[str] = "same"  # "same" = follow ``quantization``; None = keep attention projections unquantised
    weight_block_size: tuple = (128, 128)
    dtype: str = "bfloat16"

    def __post_init__(self):
        if self.v_head_dim is None:
            self.v_head_dim = self.head_dim
        if self.rotary_dim is None:
            self.rotary_dim = self.qk_rope_head_dim if self.use_mla else self.head_dim

    # ---- derived ----
    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def mla_cache_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_head_dim

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_dense_layers and (i % self.moe_layer_freq == 0)

    def layer_is_sliding(self, i: int) -> bool:
        if self.sliding_window is None:
            return False
        if self.layer_types:
            return self.layer_types[i] == "sliding_attention"
        if self.sliding_window_pattern <= 0:
            return True
        return (i + 1) % self.sliding_window_pattern != 0

    def layer_is_linear_attn(self, i: int) -> bool:
        if self.linear_attn_pattern <= 0:
            return False
        return (i + 1) % self.linear_attn_pattern != 0

    def num_params(self) -> int:
        """Rough parameter count (used for memory planning)."""
        h = self.hidden_size
        per_attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.use_mla:
            qk = self.qk_nope_head_dim + self.qk_rope_head_dim
            qa = self.q_lora_rank or 0
            per_attn = (h * (qa + self.kv_lora_rank + self.qk_rope_head_dim)
                        + qa * self.num_heads * qk
                        + self.kv_lora_rank * self.num_heads * (self.qk_nope_head_dim + self.v_head_dim)
                        + self.num_heads * self.v_head_dim * h)
        total = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        for i in range(self.num_layers):
            total += per_attn
            if self.layer_is_moe(i):
                total += self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                total += self.num_shared_experts * 3 * h * self.moe_intermediate_size
            else:
                total += 3 * h * self.intermediate_size
        return total

    @classmethod
    def from_hf_config(cls, cfg: dict) -> "ModelConfig":
        """Build from a Hugging Face ``config.json`` dict (same checkpoints the reference serves)."""
        arch = (cfg.get("architectures") or ["LlamaForCausalLM"])[0]
        if isinstance(cfg.get("thinker_config"), dict):     # Qwen3-Omni: the served part is the "thinker"
            cfg = {**cfg["thinker_config"], "architectures": [arch], "quantization_config": cfg.get("quantization_config")}
        if "hidden_size" not in cfg and "text_config" not in cfg and isinstance(cfg.get("llm_config"), dict):
            cfg = {**cfg, "text_config": cfg["llm_config"]}        # InternVL's own layout names the decoder llm_config
        if "hidden_size" not in cfg and isinstance(cfg.get("text_config"), dict):
            # nested layouts (Qwen3.5, vision-language wrappers): the decoder's fields live under text_config
            cfg = {**cfg["text_config"], **{k: v for k, v in cfg.items() if k != "text_config"},
                   "text_config": cfg["text_config"]}
        h = cfg["hidden_size"]
        nh = cfg["num_attention_heads"]
        rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
        rope = RopeScaling()
        rtype = rs.get("type", rs.get("rope_type", "none")) if rs else "none"
        if rtype in ("yarn", "deepseek_yarn"):
            rope = RopeScaling(
                type="yarn", factor=float(rs.get("factor", 1.0)),
                original_max_position=int(rs.get("original_max_position_embeddings", 4096)),
                beta_fast=float(rs.get("beta_fast", 32)), beta_slow=float(rs.get("beta_slow", 1)),
                mscale=float(rs.get("mscale", 1.0)), mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)),
                truncate=bool(rs.get("truncate", True)))
        elif rtype == "llama3":
            rope = RopeScaling(
                type="llama3", factor=float(rs.get("factor", 8.0)),
                original_max_position=int(rs.get("original_max_position_embeddings", 8192)),
                low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                high_freq_factor=float(rs.get("high_freq_factor", 4.0)))
        elif rtype == "linear":
            rope = RopeScaling(type="linear", factor=float(rs.get("factor", 1.0)))
        qc = cfg.get("quantization_config") or {}
        quant = None
        qkw: dict = {}
        wbs = (128, 128)
        if qc:
            method = qc.get("quant_method")
            if method == "fp8":
                quant = "fp8"
                wbs = tuple(qc.get("weight_block_size") or (128, 128))
            elif method in ("awq", "gptq"):
                quant = method
                qkw = {"group_size": int(qc.get("q_group_size", qc.get("group_size", 128))),
                       "bits": int(qc.get("w_bit", qc.get("bits", 4)))}
                if method == "gptq":
                    qkw["desc_act"] = bool(qc.get("desc_act", False))
            elif method == "compressed-tensors":
                quant = "int8"
                groups = qc.get("config_groups") or {}
                wq = next((g.get("weights") for g in groups.values() if isinstance(g, dict) and g.get("weights")), None)
                if isinstance(wq, dict) and int(wq.get("num_bits", 8)) == 4:      # W4A16, pack-quantized
                    quant = "w4a16"
                    qkw = {"group_size": int(wq.get("group_size") or -1), "bits": 4,
                           "symmetric": bool(wq.get("symmetric", True))}
        use_mla = "kv_lora_rank" in cfg and cfg.get("kv_lora_rank")
        kw: dict[str, Any] = dict(
            architecture=arch, name=cfg.get("_name_or_path", arch),
            vocab_size=cfg["vocab_size"], hidden_size=h, num_layers=cfg["num_hidden_layers"],
            num_heads=nh, num_kv_heads=cfg.get("num_key_value_heads", nh),
            head_dim=cfg.get("head_dim") or h // nh,
            intermediate_size=cfg.get("intermediate_size", 4 * h),
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
            # transformers 5 writes rope_theta (and partial_rotary_factor) inside rope_parameters
            rope_theta=float(cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta") or 10000.0),
            rope_scaling=rope,
            max_position=cfg.get("max_position_embeddings", 8192),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            qkv_bias=bool(cfg.get("attention_bias", arch.startswith("Qwen2"))),
            qk_norm=arch.startswith("Qwen3"),
            sliding_window=cfg.get("sliding_window") if cfg.get("use_sliding_window", True) else None,
            quantization=quant, quantization_kw=qkw, weight_block_size=wbs,
            dtype=str(cfg.get("torch_dtype", "bfloat16")),
        )
        if arch.startswith("Qwen2") or arch.startswith("Qwen3"):
            kw["sliding_window"] = None
        n_exp = cfg.get("num_experts") or cfg.get("n_routed_experts") or cfg.get("num_local_experts") or 0
        v3_like = arch in ("DeepseekV3ForCausalLM", "DeepseekV32ForCausalLM", "KimiK2ForCausalLM", "GlmMoeDsaForCausalLM")
        if n_exp:
            kw.update(
                num_experts=n_exp,
                num_experts_per_tok=cfg.get("num_experts_per_tok", 8),
                moe_intermediate_size=cfg.get("moe_intermediate_size", cfg.get("intermediate_size")),
                num_shared_experts=cfg.get("n_shared_experts", 0) or 0,
                first_dense_layers=_leading_dense(cfg),
                moe_layer_freq=cfg.get("moe_layer_freq", 1) or 1,
                # DeepSeek-V3 and its descendants score with a sigmoid and a correction bias; configs written by
                # transformers 5 no longer carry the two keys that said so
                scoring_func=cfg.get("scoring_func", "sigmoid" if v3_like else "softmax"),
                norm_topk_prob=bool(cfg.get("norm_topk_prob", True)),
                n_group=cfg.get("n_group", 1) or 1, topk_group=cfg.get("topk_group", 1) or 1,
                routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0)),
                router_bias=(cfg.get("topk_method") == "noaux_tc") if "topk_method" in cfg else v3_like,
            )
        if use_mla:
            kw.update(
                use_mla=True, q_lora_rank=cfg.get("q_lora_rank"), kv_lora_rank=cfg["kv_lora_rank"],
                qk_nope_head_dim=cfg["qk_nope_head_dim"], qk_rope_head_dim=cfg["qk_rope_head_dim"],
                v_head_dim=cfg["v_head_dim"], head_dim=cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"],
                # DeepSeek rotates q_pe / k_pe as interleaved pairs; GLM-MoE-DSA as split halves (as its indexer does)
                rope_neox=arch == "GlmMoeDsaForCausalLM" or not bool(cfg.get("rope_interleave", True)),
                index_topk=cfg.get("index_topk", 0) or 0,
                index_n_heads=cfg.get("index_n_heads", 0) or 0,
                index_head_dim=cfg.get("index_head_dim", 0) or 0,
                num_mtp_layers=cfg.get("num_nextn_predict_layers", 0) or 0,
            )
        if n_exp and cfg.get("shared_expert_intermediate_size"):
            # Qwen2-MoE / Qwen3-Next: one shared expert of its own width behind a sigmoid gate
            kw.update(num_shared_experts=1, shared_expert_gate=True,
                      shared_intermediate_size=int(cfg["shared_expert_intermediate_size"]))
        if arch == "Glm4MoeForCausalLM":
            # GLM-4.5 / 4.6 / 4.7: GQA attention with partial rotary embedding and optional per-head q / k norm,
            # DeepSeek-V3 style MoE (sigmoid scores + correction bias, grouped top-k, shared experts, dense first layers)
            kw.update(scoring_func="sigmoid", router_bias=True, qk_norm=bool(cfg.get("use_qk_norm", False)),
                      rotary_dim=int(kw["head_dim"] * float((cfg.get("rope_parameters") or {}).get("partial_rotary_factor") or cfg.get("partial_rotary_factor") or 0.5)),
                      num_mtp_layers=cfg.get("num_nextn_predict_layers", 0) or 0)
        if arch == "GptOssForCausalLM":
            kw.update(attention_sinks=True, sliding_window_pattern=2, hidden_act="swigluoai",
                      moe_bias=True, qkv_bias=True, o_bias=True,
                      sliding_window=cfg.get("sliding_window", 128))
        if arch.startswith("Qwen3Next") or arch.startswith("Qwen3_5"):
            tc = cfg.get("text_config") or cfg
            kw.update(
                linear_attn_pattern=tc.get("full_attention_interval", 4), gdn_num_k_heads=tc.get("linear_num_key_heads", 16),
                gdn_num_v_heads=tc.get("linear_num_value_heads", 32), gdn_head_k_dim=tc.get("linear_key_head_dim", 128),
                gdn_head_v_dim=tc.get("linear_value_head_dim", 128), gdn_conv_kernel=tc.get("linear_conv_kernel_dim", 4),
                attn_output_gate=True, gemma_norm=True, qk_norm=True,
                rotary_dim=int(kw["head_dim"] * float((tc.get("rope_parameters") or {}).get("partial_rotary_factor") or tc.get("partial_rotary_factor") or 0.25)),
                num_shared_experts=1 if tc.get("shared_expert_intermediate_size") else 0, shared_expert_gate=True)
        vcfg = cfg.get("vision_config")
        q35_vl = arch.startswith("Qwen3_5") and "ConditionalGeneration" in arch
        if q35_vl and not vcfg:      # a text-only export of the checkpoint: the decoder alone
            kw["architecture"] = arch = arch.replace("ForConditionalGeneration", "ForCausalLM")
            q35_vl = False
        if vcfg and ("VL" in arch or "Omni" in arch or arch.startswith("Intern") or q35_vl):
            tc = cfg.get("text_config") or cfg.get("llm_config") or cfg
            intern = arch.startswith("Intern")
            if intern:      # the transformers-native layout writes sizes as [h, w] and names the decoder by model_type
                vcfg = {**vcfg, **{k: (v[0] if isinstance(v, (list, tuple)) else v) for k, v in vcfg.items()
                                   if k in ("image_size", "patch_size")}}
                if not tc.get("architectures") and tc.get("model_type"):
                    tc = {**tc, "architectures": [{"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                                                   "llama": "LlamaForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                                                   "gpt_oss": "GptOssForCausalLM"}.get(tc["model_type"], "Qwen2ForCausalLM")]}
            kw["vision"] = dict(
                depth=vcfg.get("depth", vcfg.get("num_hidden_layers", 32)),
                hidden=vcfg.get("embed_dim", vcfg.get("hidden_size", 1280)),
                heads=vcfg.get("num_heads", vcfg.get("num_attention_heads", 16)), patch=vcfg.get("patch_size", 14),
                temporal_patch=vcfg.get("temporal_patch_size", 2), merge=vcfg.get("spatial_merge_size", 2),
                intermediate=vcfg.get("intermediate_size", int(vcfg.get("embed_dim", 1280) * vcfg.get("mlp_ratio", 4))),
                in_channels=vcfg.get("in_channels", vcfg.get("in_chans", vcfg.get("num_channels", 3))),
                norm="rmsnorm" if ("2_5" in arch or vcfg.get("norm_type") == "rms_norm") else "layernorm",
                gated_mlp="2_5" in arch, qk_norm=bool(intern and (vcfg.get("use_qk_norm") or vcfg.get("qk_normalization"))),
                act="gelu" if intern else ("gelu_tanh" if "Qwen3" in arch else "quick_gelu"), layer_scale=intern,
                image_size=vcfg.get("image_size", 448),
                # Qwen2.5-VL: windowed attention in all blocks but the listed ones (window in pixels); Qwen3-VL: a
                # learned position table interpolated to the image grid, a bias on the patch projection, exact GELU
                # in the mergers
                window_size=int(vcfg.get("window_size") or 0) if "2_5" in arch else 0,
                fullatt_blocks=list(vcfg.get("fullatt_block_indexes") or ()),
                num_pos=int(vcfg.get("num_position_embeddings") or 0) if "Qwen3" in arch else 0,
                patch_bias="Qwen3" in arch,
                downsample=cfg.get("downsample_ratio", 0.5), image_token_id=cfg.get("image_token_id", 151655),
                # videos: Qwen2.5-VL spaces temporal positions by seconds x tokens_per_second; Qwen3-VL prompts hold
                # one placeholder run per temporal patch
                video_token_id=cfg.get("video_token_id"),
                tokens_per_second=(vcfg.get("tokens_per_second", 4) if "2_5" in arch else
                                   cfg.get("position_id_per_seconds", 25) if "Omni" in arch else 0),
                video_frame_runs="Qwen3VL" in arch or q35_vl,
                text_architecture=(tc.get("architectures") or ["Qwen2ForCausalLM"])[0] if intern else
                (arch.replace("ForConditionalGeneration", "ForCausalLM") if q35_vl else
                 "Qwen3MoeForCausalLM" if ("Qwen3" in arch and "Moe" in arch) else
                 "Qwen3ForCausalLM" if "Qwen3" in arch else "Qwen2ForCausalLM"),
                deepstack_indexes=list(vcfg.get("deepstack_visual_indexes", ())))
            acfg = cfg.get("audio_config")
            if acfg and "Omni" in arch:
                kw["vision"]["audio"] = dict(
                    hidden=acfg.get("d_model", 1280), heads=acfg.get("encoder_attention_heads", 20),
                    intermediate=acfg.get("encoder_ffn_dim", 5120), depth=acfg.get("encoder_layers", 32),
                    n_mels=acfg.get("num_mel_bins", 128), n_window=acfg.get("n_window", 50),
                    n_window_infer=acfg.get("n_window_infer", 400), conv_chunksize=acfg.get("conv_chunksize", 500),
                    downsample_hidden=acfg.get("downsample_hidden_size", 480))
                kw["vision"]["audio_token_id"] = cfg.get("audio_token_id", 151646)
            rsc = tc.get("rope_scaling") or tc.get("rope_parameters") or {}
            kw["mrope_section"] = tuple(rsc.get("mrope_section", ()))
            # Qwen3-VL interleaves the three position axes over the rotary pairs (t h w t h w ...); Qwen2-VL / 2.5-VL
            # give each axis a contiguous section
            kw["mrope_interleaved"] = bool(rsc.get("mrope_interleaved", arch.startswith("Qwen3VL") or arch.startswith("Qwen3Omni") or q35_vl))
        if vcfg and arch.startswith("Gemma"):
            rp = vcfg.get("rope_parameters") or {}
            kw["vision"] = dict(
                depth=vcfg.get("num_hidden_layers", 16), hidden=vcfg.get("hidden_size", 768),
                heads=vcfg.get("num_attention_heads", 12), kv_heads=vcfg.get("num_key_value_heads"),
                head_dim=vcfg.get("head_dim"), patch=vcfg.get("patch_size", 16),
                intermediate=vcfg.get("intermediate_size", 3072), in_channels=3,
                position_embedding_size=vcfg.get("position_embedding_size", 10240),
                pool=vcfg.get("pooling_kernel_size", 3), standardize=bool(vcfg.get("standardize")),
                eps=vcfg.get("rms_norm_eps", 1e-6), rope_theta=float(rp.get("rope_theta", 100.0)),
                image_token_id=cfg.get("image_token_id", 258880), text_architecture="Gemma4ForCausalLM",
                pad_token_id=int((cfg.get("text_config") or {}).get("pad_token_id") or 0))
        if arch.startswith("Gemma"):
            kw.update(num_kv_shared_layers=cfg.get("num_kv_shared_layers", 0) or 0,
                      final_logit_softcapping=float(cfg.get("final_logit_softcapping") or 0.0),
                      attn_scale=(float(cfg["query_pre_attn_scalar"]) ** -0.5 if cfg.get("query_pre_attn_scalar") else None),
                      per_layer_input_size=int(cfg.get("hidden_size_per_layer_input") or 0),
                      per_layer_vocab_size=int(cfg.get("vocab_size_per_layer_input") or cfg.get("vocab_size") or 0))
            kw.update(gemma_norm=True, hidden_act="gelu_tanh", qk_norm=True,
                      sliding_window=cfg.get("sliding_window"), sliding_window_pattern=cfg.get("sliding_window_pattern", 6),
                      tie_word_embeddings=True)
            if arch.startswith("Gemma4"):
                # sparse block beside the dense MLP of every layer (26B-A4B): top_k_experts of num_experts
                if cfg.get("enable_moe_block") and cfg.get("num_experts"):
                    kw.update(num_experts=int(cfg["num_experts"]), num_experts_per_tok=int(cfg.get("top_k_experts") or 8),
                              moe_intermediate_size=int(cfg.get("moe_intermediate_size") or cfg["intermediate_size"]),
                              first_dense_layers=0, moe_layer_freq=1, scoring_func="softmax", norm_topk_prob=True)
                else:
                    kw["num_experts"] = 0
                # Gemma-4: norm weights multiply directly (no 1 + w), softmax scale 1 (q / k are normalised), V is
                # RMS-normalised, a scalar per layer, rotary parameters per layer type ("proportional" on the full-
                # attention layers: only a fraction of the angle pairs rotates)
                rp = cfg.get("rope_parameters") or {}
                per_type = {}
                for lt, key in (("sliding_attention", "sliding"), ("full_attention", "full")):
                    r = rp.get(lt) if isinstance(rp.get(lt), dict) else None
                    if r:
                        sc = RopeScaling(type="proportional", partial=float(r.get("partial_rotary_factor", 1.0)),
                                         factor=float(r.get("factor", 1.0))) if r.get("rope_type") == "proportional" else RopeScaling()
                        per_type[key] = (float(r.get("rope_theta", 10000.0)), sc)
                kw.update(gemma_norm=False, attn_scale=1.0, v_norm=True, layer_scalar=True, rope_per_type=per_type,
                          layer_types=tuple(cfg.get("layer_types") or ()),
                          double_wide_mlp=bool(cfg.get("use_double_wide_mlp", False)),
                          global_head_dim=cfg.get("global_head_dim") or None,
                          attention_k_eq_v=bool(cfg.get("attention_k_eq_v", False)),
                          num_global_kv_heads=cfg.get("num_global_key_value_heads") or None)
        if arch == "MiMoV2FlashForCausalLM":
            kw.update(v_head_dim=cfg.get("v_head_dim", kw["head_dim"]), attention_sinks=bool(cfg.get("add_swa_attention_sink_bias", True)),
                      sliding_window=cfg.get("sliding_window", 128), sliding_window_pattern=cfg.get("hybrid_block_size", 0) or 0)
        out = cls(**kw)
        if arch.startswith("Intern") and isinstance(cfg.get("text_config") or cfg.get("llm_config"), dict):
            # the decoder's traits (q/k/v biases, q/k norms, routing, ...) follow ITS architecture, not the wrapper's
            tcfg = dict(cfg.get("text_config") or cfg.get("llm_config"))
            tcfg["architectures"] = [out.vision["text_architecture"]]
            tcfg.setdefault("torch_dtype", cfg.get("torch_dtype", "bfloat16"))
            if cfg.get("quantization_config") and not tcfg.get("quantization_config"):
                tcfg["quantization_config"] = cfg["quantization_config"]
            text = cls.from_hf_config(tcfg)
            text.architecture, text.name, text.vision = arch, out.name, out.vision
            text.tie_word_embeddings = out.tie_word_embeddings
            return text
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_config(json.load(f))


def _leading_dense(cfg: dict) -> int:
    """Number of dense MLP layers in front of the MoE layers: ``first_k_dense_replace``, or the leading ``"dense"``
    entries of ``mlp_layer_types`` (how configs written by transformers 5 spell it)."""
    types = cfg.get("mlp_layer_types")
    if isinstance(types, (list, tuple)) and types:
        n = 0
        while n < len(types) and types[n] == "dense":
            n += 1
        return n
    return cfg.get("first_k_dense_replace", 0) or 0


@dataclass
class CacheConfig:
    block_size: int = 16
    num_blocks: Optional[int] = None  # None = derive from memory budget
    gpu_memory_utilization: float = 0.9
    cache_dtype: str = "auto"  # "auto" | "bfloat16" | "fp8_ds_mla"
    enable_prefix_caching: bool = False


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    use_sequence_parallel_moe: bool = False
    fused_collectives: bool = True  # GEMM+reduce-scatter / all-gather+GEMM kernels when peers are mapped

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size * self.pipeline_parallel_size


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 8192
    enable_chunked_prefill: bool = True


@dataclass
class SpeculativeConfig:
    method: Optional[str] = None  # None | "mtp" | "eagle" | "eagle3" | "ngram"
    num_speculative_tokens: int = 0
    ngram_n: int = 3
    draft_weights_path: Optional[str] = None  # safetensors directory of the draft model (random init when absent)


@dataclass
class CompilationConfig:
    """CUDA-graph settings.  The reference only supports piecewise graphs
    (``docs/source/developer_guide/feature_guide/Kunlun_Graph.md:58-75``); here the
    decode step is captured whole, and ``piecewise`` keeps attention outside."""

    mode: str = "full_decode"  # "none" | "piecewise" | "full_decode"
    capture_sizes: tuple = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


@dataclass
class LoRAConfig:
    enable: bool = False
    max_loras: int = 4
    max_lora_rank: int = 16


@dataclass
class EngineConfig:
    model: ModelConfig
    cache: CacheConfig = field(default_factory=CacheConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    compilation: CompilationConfig = field(default_factory=CompilationConfig)
    lora: LoRAConfig = field(default_factory=LoRAConfig)
    device: str = "cpu"
    seed: int = 0
    weights_path: Optional[str] = None
    init_std: float = 0.02

    def finalize(self) -> "EngineConfig":
        """Apply the platform fix-ups the reference performs in
        ``check_and_update_config`` (``platforms/kunlun.py:147-245``)."""
        m = self.model
        if m.use_mla and self.cache.block_size not in (64,):
            self.cache.block_size = 64
        if m.index_topk and self.cache.cache_dtype == "auto":
            self.cache.cache_dtype = "bfloat16"
        if self.device == "cpu":
            self.compilation.mode = "none"
        if m.linear_attn_pattern:
            # the recurrent state of a cached prefix is not kept, and a rejected draft cannot be rolled back
            self.cache.enable_prefix_caching = False
            if self.speculative.num_speculative_tokens:
                raise ValueError("speculative decoding is not supported with linear-attention layers")
        if self.speculative.method == "eagle3":
            self.compilation.mode = "none"  # the auxiliary hidden states are not carried through captured graphs
        if self.speculative.method == "mtp" and not m.num_mtp_layers:
            raise ValueError("MTP speculative decoding needs a model with MTP layers")
        self.scheduler.max_num_batched_tokens = max(
            self.scheduler.max_num_batched_tokens, self.cache.block_size)
        return self


# --------------------------------------------------------------------------------------
# Presets: the architectures named by the benchmark configurations.
# --------------------------------------------------------------------------------------

def qwen2_0_5b() -> ModelConfig:
    return ModelConfig(
        architecture="Qwen2ForCausalLM", name="qwen2-0.5b", vocab_size=151936, hidden_size=896,
        num_layers=24, num_heads=14, num_kv_heads=2, head_dim=64, intermediate_size=4864,
        rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True, qkv_bias=True,
        max_position=32768, dtype="float32")


def llama_3_1_8b() -> ModelConfig:
    return ModelConfig(
        architecture="LlamaForCausalLM", name="llama-3.1-8b", vocab_size=128256, hidden_size=4096,
        num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336,
        rms_norm_eps=1e-5, rope_theta=5e5, max_position=131072)


def qwen3_8b() -> ModelConfig:
    return ModelConfig(
        architecture="Qwen3ForCausalLM", name="qwen3-8b", vocab_size=151936, hidden_size=4096,
        num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=12288,
        rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, max_position=40960)


def qwen3_next_80b_a3b() -> ModelConfig:
    return ModelConfig(
        architecture="Qwen3NextForCausalLM", name="qwen3-next-80b-a3b", vocab_size=151936, hidden_size=2048,
        num_layers=48, num_heads=16, num_kv_heads=2, head_dim=256, intermediate_size=5120, rms_norm_eps=1e-6,
        rope_theta=1e7, rotary_dim=64, qk_norm=True, gemma_norm=True, attn_output_gate=True, max_position=262144,
        num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512, num_shared_experts=1,
        shared_expert_gate=True, norm_topk_prob=True, linear_attn_pattern=4, gdn_num_k_heads=16, gdn_num_v_heads=32,
        gdn_head_k_dim=128, gdn_head_v_dim=128, gdn_conv_kernel=4)


def qwen3_30b_a3b(fp8: bool = True) -> ModelConfig:
    return ModelConfig(
        architecture="Qwen3MoeForCausalLM", name="qwen3-30b-a3b", vocab_size=151936, hidden_size=2048,
        num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128, intermediate_size=6144,
        rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, num_experts=128, num_experts_per_tok=8,
        moe_intermediate_size=768, scoring_func="softmax", norm_topk_prob=True,
        max_position=40960, quantization="fp8" if fp8 else None)


def deepseek_v3(fp8: bool = True, sparse: bool = False) -> ModelConfig:
    return ModelConfig(
        architecture="DeepseekV32ForCausalLM" if sparse else "DeepseekV3ForCausalLM",
        name="deepseek-v3.2" if sparse else "deepseek-v3", vocab_size=129280, hidden_size=7168,
        num_layers=61, num_heads=128, num_kv_heads=128, head_dim=192, v_head_dim=128,
        intermediate_size=18432, rms_norm_eps=1e-6, rope_theta=10000.0, rope_neox=False,
        rope_scaling=RopeScaling(type="yarn", factor=40.0, original_max_position=4096,
                                 beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0),
        use_mla=True, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
        num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048, num_shared_experts=1,
        first_dense_layers=3, scoring_func="sigmoid", norm_topk_prob=True, n_group=8, topk_group=4,
        routed_scaling_factor=2.5, router_bias=True, num_mtp_layers=1, max_position=163840,
        index_topk=2048 if sparse else 0, index_n_heads=64 if sparse else 0,
        index_head_dim=128 if sparse else 0, quantization="fp8" if fp8 else None)


def gpt_oss_20b() -> ModelConfig:
    return ModelConfig(
        architecture="GptOssForCausalLM", name="gpt-oss-20b", vocab_size=201088, hidden_size=2880,
        num_layers=24, num_heads=64, num_kv_heads=8, head_dim=64, intermediate_size=2880,
        rms_norm_eps=1e-5, rope_theta=150000.0, qkv_bias=True, o_bias=True, num_experts=32,
        num_experts_per_tok=4, moe_intermediate_size=2880, scoring_func="softmax_after_topk",
        hidden_act="swigluoai", moe_bias=True, attention_sinks=True, sliding_window=128,
        sliding_window_pattern=2, max_position=131072)


PRESETS = {
    "qwen2-0.5b": qwen2_0_5b,
    "llama-3.1-8b": llama_3_1_8b,
    "qwen3-8b": qwen3_8b,
    "qwen3-30b-a3b": qwen3_30b_a3b,
    "qwen3-next-80b-a3b": qwen3_next_80b_a3b,
    "deepseek-v3": deepseek_v3,
    "deepseek-v3.2": lambda: deepseek_v3(sparse=True),
    "gpt-oss-20b": gpt_oss_20b,
}


def tiny(base: ModelConfig, **overrides) -> ModelConfig:
    """Shrink a preset for tests while keeping its structure (derived head sizes are re-derived)."""
    if "head_dim" in overrides and not base.use_mla:
        overrides.setdefault("v_head_dim", None)
        overrides.setdefault("rotary_dim", None)
    return dataclasses.replace(base, **overrides)


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return cdiv(a, b) * b


def yarn_mscale(scale: float, mscale: float) -> float:
    if scale <= 1.0:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0
