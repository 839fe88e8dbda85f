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

    # Decode-sized calls of SMALL projections (attention q/k/v/o of the MoE models) are latency-bound, and the fp8
    # kernel has no split-K: with M <= 64 tokens a [2048 x 4096] weight gives it 16 tiles for 148 SMs.  Such layers
    # keep a second, 16-bit copy of the weight (de-quantised once) and send small batches through the 16-bit
    # stream-K GEMM - which also skips the activation quantiser.  Large batches stay on the fp8 tensor-core path.
    SMALL_WEIGHT_ELEMS = 48 << 20
    SMALL_BATCH_ROWS = 64

    def apply(self, layer, x: torch.Tensor) -> torch.Tensor:
        w16 = getattr(layer, "weight_16bit", None)
        if w16 is not None and x.is_cuda and x.numel() // x.shape[-1] <= self.SMALL_BATCH_ROWS:
            return ops.linear(x, w16, layer.bias)
        return ops.fp8_linear(x, layer.weight, layer.weight_scale_inv, layer.bias, self.block, layer.out_dtype)

    def process_weights_after_loading(self, layer):
        w = layer.weight
        if (w.is_cuda and w.numel() <= self.SMALL_WEIGHT_ELEMS and layer.out_dtype in (torch.bfloat16, torch.float16)
                and w.shape[1] % 8 == 0):
            bn, bk = self.block
            s = layer.weight_scale_inv.data
            sf = s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
            layer.weight_16bit = (w.data.float() * sf).to(layer.out_dtype)

    @staticmethod
    def quantize_(layer, w: torch.Tensor, block=(128, 128)):
        """Random-init / bf16-checkpoint path: quantise ``w`` per 128x128 absmax into the layer."""
        q, s = ops.reference_basic.quant_fp8_block(w.float().cpu(), block)
        layer.weight.data.copy_(q.to(layer.weight.device))
        layer.weight_scale_inv.data.copy_(s.to(layer.weight.device))
