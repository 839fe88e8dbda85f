"""fp8 e4m3 linear with 128x128 weight block scales and dynamic 1x128 activation scales.

Checkpoint contract: ``weight`` is ``float8_e4m3fn [N, K]`` and ``weight_scale_inv`` is
``float32 [ceil(N/128), ceil(K/128)]`` with ``w ~= weight * weight_scale_inv[block]``.  Sharding a
merged / row-parallel layer shards the scale tensor by ``ceil(offset / 128)`` rows or columns - the
rule the reference implements in ``adjust_block_scale_shard`` (``ops/linear.py:91-96,246-250,385-407``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config import cdiv
from ..models.layers import param


class Fp8BlockLinearMethod:
    name = "fp8"

    def __init__(self, block=(128, 128)):
        self.block = tuple(block)

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        bn, bk = self.block
        layer.weight = param(out_local, in_local, dtype=torch.float8_e4m3fn, device=device)
        layer.weight_scale_inv = param(cdiv(out_local, bn), cdiv(in_local, bk), dtype=torch.float32, device=device)
        layer.out_dtype = dtype

    def aux_params(self):
        return {"weight_scale_inv": self.block}

    def apply(self, layer, x: torch.Tensor) -> torch.Tensor:
        # decode-sized batches (<= 32 rows) run on the cluster split-K fp8 kernel, larger ones on the grouped
        # block-scaled kernel; both read the fp8 weight itself, so no 16-bit copy of it is kept
        return ops.fp8_linear(x, layer.weight, layer.weight_scale_inv, layer.bias, self.block, layer.out_dtype)

    def process_weights_after_loading(self, layer):
        return None

    @staticmethod
    def quantize_(layer, w: torch.Tensor, block=(128, 128)):
        """Random-init / bf16-checkpoint path: quantise ``w`` per 128x128 absmax into the layer."""
        q, s = ops.reference_basic.quant_fp8_block(w.float().cpu(), block)
        layer.weight.data.copy_(q.to(layer.weight.device))
        layer.weight_scale_inv.data.copy_(s.to(layer.weight.device))
