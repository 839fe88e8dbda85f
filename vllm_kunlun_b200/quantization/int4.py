"""AWQ / GPTQ 4-bit weight-only linears.

Reference: ``quantization/awq.py:124-168`` (repack at load, dequant+matmul for >= 256 tokens, fused
gemm below) and ``quantization/gptq.py:68-143`` (exllama-style shuffle + gemm).  Here the packed
tensors are unpacked ONCE after loading into a bf16 weight in the GEMM's layout (K-major rows), so
the hot path is the same tcgen05 GEMM as for unquantised layers; the packed tensors are dropped."""
from __future__ import annotations

import torch

from .. import ops
from ..models.layers import param
from ..ops.reference import basic as rb


class AWQLinearMethod:
    name = "awq"

    def __init__(self, group_size: int = 128, bits: int = 4):
        self.group_size, self.bits = group_size, bits

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        g = self.group_size if self.group_size > 0 else in_local
        layer.qweight = param(in_local, out_local // 8, dtype=torch.int32, device=device)
        layer.qzeros = param(in_local // g, out_local // 8, dtype=torch.int32, device=device)
        layer.scales = param(in_local // g, out_local, dtype=dtype, device=device)
        layer.weight = None

    def aux_params(self):
        return {}

    def process_weights_after_loading(self, layer):
        if layer.qweight is None:
            return
        g = self.group_size if self.group_size > 0 else layer.qweight.shape[0]
        w = rb.awq_dequantize(layer.qweight.data.cpu(), layer.scales.data.cpu(), layer.qzeros.data.cpu(), g)
        layer.weight = torch.nn.Parameter(w.T.contiguous().to(layer.scales.device), requires_grad=False)
        layer.qweight = layer.qzeros = None

    def apply(self, layer, x):
        return ops.linear(x, layer.weight, layer.bias)


class GPTQLinearMethod:
    name = "gptq"

    def __init__(self, group_size: int = 128, bits: int = 4, desc_act: bool = False):
        self.group_size, self.bits, self.desc_act = group_size, bits, desc_act

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        pack = 32 // self.bits
        g = self.group_size if self.group_size > 0 else in_local
        layer.qweight = param(in_local // pack, out_local, dtype=torch.int32, device=device)
        layer.qzeros = param(in_local // g, out_local // pack, dtype=torch.int32, device=device)
        layer.scales = param(in_local // g, out_local, dtype=dtype, device=device)
        layer.g_idx = param(in_local, dtype=torch.int32, device=device)
        layer.g_idx.data.copy_(torch.arange(in_local, dtype=torch.int32) // g)
        layer.weight = None

    def aux_params(self):
        return {}

    def process_weights_after_loading(self, layer):
        if layer.qweight is None:
            return
        w = rb.gptq_dequantize(layer.qweight.data.cpu(), layer.scales.data.cpu(), layer.qzeros.data.cpu(),
                               layer.g_idx.data.cpu(), self.bits)
        layer.weight = torch.nn.Parameter(w.T.contiguous().to(layer.scales.device), requires_grad=False)
        layer.qweight = layer.qzeros = None

    def apply(self, layer, x):
        return ops.linear(x, layer.weight, layer.bias)
