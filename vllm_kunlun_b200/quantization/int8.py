"""compressed-tensors W8A8 int8 (dynamic per-token or static per-tensor activations, per-channel weights).

Reference: ``quantization/compressed_tensors/compressed_tensors.py:47-82`` and the scaled-mm kernel
wrapper ``quantization/kernels/scale_mm.py:43-90`` (which converts scales to the device's "max"
convention, ``* 127``; this implementation keeps plain scales)."""
from __future__ import annotations

import torch

from .. import ops
from ..models.layers import param


class Int8LinearMethod:
    name = "int8"

    def __init__(self, static_input_scale: bool = False):
        self.static = static_input_scale

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        layer.weight = param(out_local, in_local, dtype=torch.int8, device=device)
        layer.weight_scale = param(out_local, 1, dtype=torch.float32, device=device)
        layer.input_scale = param(1, dtype=torch.float32, device=device) if self.static else None
        layer.out_dtype = dtype

    def aux_params(self):
        return {"weight_scale": (1, 1)}

    def apply(self, layer, x):
        return ops.int8_linear(x, layer.weight, layer.weight_scale, layer.bias, layer.input_scale, layer.out_dtype)

    def process_weights_after_loading(self, layer):
        pass

    @staticmethod
    def quantize_(layer, w: torch.Tensor):
        wf = w.float()
        s = wf.abs().amax(-1, keepdim=True).clamp(min=1e-8) / 127.0
        layer.weight.data.copy_(torch.round(wf / s).clamp(-128, 127).to(torch.int8))
        layer.weight_scale.data.copy_(s)
