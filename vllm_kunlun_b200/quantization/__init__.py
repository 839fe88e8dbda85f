"""Quantization methods.

The reference re-registers ``awq``, ``gptq`` and ``compressed-tensors`` (W8A8 int8 dynamic / static,
W4A16) with its own kernels (``vllm_kunlun/quantization/*``) and has **no fp8 compute** (fp8 is not in
its dtype whitelist, ``platforms/kunlun.py:349-364``).  This package provides the same int8 / int4
checkpoint formats plus fp8 e4m3 with 128x128 block scales (``weight_scale_inv`` tensors), the
format of the DeepSeek-V3 / Qwen3-MoE fp8 checkpoints.
"""
from ..models.layers import register_linear_method
from .fp8 import Fp8BlockLinearMethod
from .int4 import AWQLinearMethod, CompressedTensorsW4A16LinearMethod, GPTQLinearMethod
from .int8 import Int8LinearMethod

register_linear_method("fp8", Fp8BlockLinearMethod)
register_linear_method("int8", Int8LinearMethod)
register_linear_method("awq", AWQLinearMethod)
register_linear_method("gptq", GPTQLinearMethod)
register_linear_method("w4a16", CompressedTensorsW4A16LinearMethod)

QUANTIZATION_METHODS = ["fp8", "int8", "compressed-tensors", "awq", "gptq"]
