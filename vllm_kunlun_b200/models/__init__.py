"""Model registry.

The reference registers ~20 architectures with ``ModelRegistry.register_model(arch, "module:Class")``
(``vllm_kunlun/models/__init__.py:4-113``).  The same architecture strings resolve here, lazily,
to this framework's model classes.
"""
from __future__ import annotations

import importlib

from ..config import ModelConfig

_REGISTRY = {
    # dense GQA decoders (upstream model files in the reference; native here)
    "LlamaForCausalLM": "dense:DenseForCausalLM",
    "MistralForCausalLM": "dense:DenseForCausalLM",
    "Qwen2ForCausalLM": "dense:DenseForCausalLM",
    "Qwen3ForCausalLM": "dense:DenseForCausalLM",
    "InternLM2ForCausalLM": "dense:DenseForCausalLM",
    "SeedOssForCausalLM": "dense:DenseForCausalLM",
    # MoE
    "Qwen3MoeForCausalLM": "moe:MoEForCausalLM",
    "Qwen2MoeForCausalLM": "moe:MoEForCausalLM",
    "GptOssForCausalLM": "gpt_oss:GptOssForCausalLM",
    "MixtralForCausalLM": "moe:MoEForCausalLM",
    # MLA family
    "DeepseekV2ForCausalLM": "deepseek:DeepseekForCausalLM",
    "DeepseekV3ForCausalLM": "deepseek:DeepseekForCausalLM",
    "DeepseekV32ForCausalLM": "deepseek:DeepseekForCausalLM",
    "GlmMoeDsaForCausalLM": "deepseek:DeepseekForCausalLM",
    "Glm4MoeForCausalLM": "deepseek:DeepseekForCausalLM",     # GQA attention + DeepSeek-V3 style MoE
    "KimiK2ForCausalLM": "deepseek:DeepseekForCausalLM",
    "DeepSeekMTPModel": "deepseek_mtp:DeepSeekMTP",
    # hybrid linear attention
    "Qwen3NextForCausalLM": "qwen3_next:Qwen3NextForCausalLM",
    "Qwen3_5ForConditionalGeneration": "vision:Qwen3_5ForConditionalGeneration",
    "Qwen3_5MoeForConditionalGeneration": "vision:Qwen3_5ForConditionalGeneration",
    "Qwen3_5ForCausalLM": "qwen3_next:Qwen3NextForCausalLM",          # the text-only classes of the same checkpoints
    "Qwen3_5MoeForCausalLM": "qwen3_next:Qwen3NextForCausalLM",
    # asymmetric V / sliding window with sinks
    "MiMoV2FlashForCausalLM": "mimo_v2_flash:MiMoV2FlashForCausalLM",
    # Gemma family
    "Gemma4ForCausalLM": "gemma4:Gemma4ForCausalLM",
    "Gemma4ForConditionalGeneration": "vision:Gemma4ForConditionalGeneration",
    # vision-language wrappers (ViT tower + a registered text decoder)
    "Qwen2VLForConditionalGeneration": "vision:QwenVLForConditionalGeneration",
    "Qwen2_5_VLForConditionalGeneration": "vision:QwenVLForConditionalGeneration",
    "Qwen3VLForConditionalGeneration": "vision:QwenVLForConditionalGeneration",
    "Qwen3VLMoeForConditionalGeneration": "vision:Qwen3VLMoeForConditionalGeneration",
    "Qwen3OmniMoeForConditionalGeneration": "omni:Qwen3OmniMoeThinker",
    "Qwen3OmniMoeThinkerForConditionalGeneration": "omni:Qwen3OmniMoeThinker",
    "InternVLChatModel": "vision:InternVLChatModel",
    "InternVLForConditionalGeneration": "vision:InternVLChatModel",
    "InternS1ForConditionalGeneration": "vision:InternVLChatModel",
}


def register_model(arch: str, target: str) -> None:
    """``target`` is ``"module:Class"`` relative to this package or an absolute ``pkg.mod:Class``."""
    _REGISTRY[arch] = target


def supported_architectures() -> list:
    return sorted(_REGISTRY)


def resolve_model_cls(arch: str):
    if arch not in _REGISTRY:
        raise ValueError(f"unsupported architecture {arch!r}; known: {supported_architectures()}")
    mod, cls = _REGISTRY[arch].split(":")
    module = importlib.import_module(mod if "." in mod else f"{__name__}.{mod}")
    return getattr(module, cls)


def build_model(cfg: ModelConfig, device="cpu", dtype=None):
    if cfg.quantization and cfg.quantization_kw:      # group size, bits, ... of the checkpoint's quantization_config
        from .layers import set_quant_defaults
        set_quant_defaults(cfg.quantization, cfg.quantization_kw)
    return resolve_model_cls(cfg.architecture)(cfg, device=device, dtype=dtype)
