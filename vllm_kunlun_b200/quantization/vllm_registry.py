"""Quantization configs registered with upstream vLLM's quantization registry.

Reference: the plugin re-registers ``awq``, ``gptq`` and ``compressed-tensors`` with ``@register_quantization_config``
(``quantization/awq.py:40``, ``gptq.py:47``, ``compressed_tensors/compressed_tensors.py:47``) so that upstream's
layers call its kernels.  The reference has no fp8 compute at all (fp8 is not in its dtype whitelist,
``platforms/kunlun.py:349-364``); here the fp8 block-128 format (``weight`` e4m3 + ``weight_scale_inv`` fp32 per
128x128 block, activations quantised per 1x128 group on the fly) is the one that is registered, under upstream's
name ``fp8``, so that DeepSeek-V3 / Qwen3 fp8 checkpoints run on the tcgen05 block-scaled GEMM under upstream's engine.

``register_quant_configs()`` is idempotent and a no-op when vLLM is not importable.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from .. import ops

_DONE = [False]
REGISTERED: dict = {}


def register_quant_configs() -> dict:
    if _DONE[0]:
        return REGISTERED
    try:
        from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
        from vllm.model_executor.layers.quantization import register_quantization_config
        from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
        from vllm.model_executor.parameter import BlockQuantScaleParameter, ModelWeightParameter
    except Exception:
        return REGISTERED
    _DONE[0] = True

    class B200Fp8LinearMethod(LinearMethodBase):
        """Block-scaled fp8 linear on ``ops.fp8_linear`` (tcgen05 ``kind::f8f6f4`` with software scale promotion)."""

        def __init__(self, quant_config: "B200Fp8Config"):
            self.quant_config = quant_config
            self.block = tuple(quant_config.weight_block_size)

        def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list,
                           input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
            out = sum(output_partition_sizes)
            bn, bk = self.block
            loader = extra_weight_attrs.get("weight_loader")
            for n in output_partition_sizes[:-1]:
                if n % bn:
                    raise ValueError(f"merged output partition of {n} rows is not a multiple of the {bn}-row scale block")
            layer.logical_widths = output_partition_sizes
            layer.input_size_per_partition = input_size_per_partition
            layer.output_size_per_partition = out
            layer.orig_dtype = params_dtype
            layer.weight_block_size = list(self.block)
            w = ModelWeightParameter(data=torch.empty(out, input_size_per_partition, dtype=torch.float8_e4m3fn),
                                     input_dim=1, output_dim=0, weight_loader=loader)
            layer.register_parameter("weight", w)
            s = BlockQuantScaleParameter(
                data=torch.empty(-(-out // bn), -(-input_size_per_partition // bk), dtype=torch.float32),
                input_dim=1, output_dim=0, weight_loader=loader)
            s[:] = torch.finfo(torch.float32).min
            layer.register_parameter("weight_scale_inv", s)  # the checkpoint's name, as DeepSeek-V3 stores it

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            layer.weight = torch.nn.Parameter(layer.weight.data.contiguous(), requires_grad=False)
            layer.weight_scale_inv = torch.nn.Parameter(layer.weight_scale_inv.data.contiguous(), requires_grad=False)

        def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
            return ops.fp8_linear(x, layer.weight, layer.weight_scale_inv, bias, self.block,
                                  x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16)

    @register_quantization_config("fp8")
    class B200Fp8Config(QuantizationConfig):
        """``quant_method: fp8`` with ``weight_block_size: [128, 128]`` and dynamic activations."""

        def __init__(self, weight_block_size=(128, 128), ignored_layers: Optional[list] = None):
            super().__init__()
            self.weight_block_size = list(weight_block_size)
            self.ignored_layers = ignored_layers or []

        def get_name(self) -> str:
            return "fp8"

        def get_supported_act_dtypes(self) -> list:
            return [torch.bfloat16, torch.float16]

        @classmethod
        def get_min_capability(cls) -> int:
            return 100

        @staticmethod
        def get_config_filenames() -> list:
            return []

        @classmethod
        def from_config(cls, config: dict) -> "B200Fp8Config":
            fmt = config.get("fmt", "e4m3")
            if fmt != "e4m3":
                raise ValueError(f"fp8 format {fmt!r}: only e4m3 weights are served")
            act = config.get("activation_scheme", "dynamic")
            if act != "dynamic":
                raise ValueError("only dynamic (per 1x128 group) activation quantisation is served")
            block = config.get("weight_block_size")
            if not block or list(block) != [128, 128]:
                raise ValueError(f"weight_block_size={block!r}: the block-scaled GEMM serves 128x128 weight blocks")
            return cls(block, config.get("ignored_layers") or config.get("modules_to_not_convert"))

        def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> Optional[Any]:
            if isinstance(layer, LinearBase):
                if any(prefix == n or prefix.endswith("." + n) or n in prefix for n in self.ignored_layers):
                    return UnquantizedLinearMethod()
                return B200Fp8LinearMethod(self)
            return None

    REGISTERED["fp8"] = B200Fp8Config
    REGISTERED["fp8_linear_method"] = B200Fp8LinearMethod
    return REGISTERED
