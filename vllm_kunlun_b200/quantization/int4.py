"""AWQ / GPTQ 4-bit weight-only linears.

Reference: ``quantization/awq.py:124-168`` (repack at load, dequant+matmul for >= 256 tokens, fused
gemm below) and ``quantization/gptq.py:68-143`` (exllama-style shuffle + gemm).

After loading, the checkpoint's packed tensors are repacked ONCE into the layout the kernels read
(``pack_w4``: one row of ``K / 2`` bytes per output feature, k contiguous) together with
``scale`` / ``zero`` as ``[N, K / group]``; nothing 16-bit is kept.  Decode-sized batches (<= 32 rows)
stream the packed bytes and de-quantise inside the tcgen05 GEMM (``csrc/gemm/gemm_decode.cu``: a
quarter of the 16-bit weight bytes per step); larger batches de-quantise into a temporary and run the
16-bit GEMM.  Layers the packed kernels do not take (group sizes that are not a multiple of 64,
GPTQ ``desc_act`` with a permuted ``g_idx``, K not a multiple of the group) fall back to a 16-bit
weight built at load time."""
from __future__ import annotations

import torch

from .. import ops
from ..models.layers import param
from ..ops.reference import basic as rb

# nibble position of the e-th of the eight consecutive k values a 32-bit word holds: the kernel extracts the pair
# (2 j, 2 j + 1) as ``(w >> 4 j) & 0x000F000F``
_NIBBLE_POS = (0, 4, 1, 5, 2, 6, 3, 7)


def pack_w4(q: torch.Tensor) -> torch.Tensor:
    """``q [N, K]`` integer values in 0..15 -> ``uint8 [N, K / 2]`` in the kernels' layout."""
    N, K = q.shape
    assert K % 8 == 0
    v = q.reshape(N, K // 8, 8).to(torch.int64) & 0xF
    word = torch.zeros(N, K // 8, dtype=torch.int64, device=q.device)
    for e, pos in enumerate(_NIBBLE_POS):
        word |= v[..., e] << (4 * pos)
    b = torch.stack([(word >> (8 * i)) & 0xFF for i in range(4)], -1)       # little-endian bytes of each word
    return b.to(torch.uint8).reshape(N, K // 2).contiguous()


def unpack_w4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of ``pack_w4``: ``uint8 [N, K / 2]`` -> ``int32 [N, K]`` values in 0..15."""
    N, half = packed.shape
    b = packed.reshape(N, half // 4, 4).to(torch.int64)
    word = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    v = torch.stack([(word >> (4 * pos)) & 0xF for pos in _NIBBLE_POS], -1)
    return v.reshape(N, half * 2).to(torch.int32)


def dequant_w4(packed, scale, zero, group: int) -> torch.Tensor:
    """Oracle: ``W[n, k] = (q[n, k] - zero[n, k / group]) * scale[n, k / group]`` rounded once to the scale dtype."""
    q = unpack_w4(packed).float()
    z = zero.float().repeat_interleave(group, 1)
    s = scale.float().repeat_interleave(group, 1)
    return ((q - z) * s).to(scale.dtype)


def packed_ok(K: int, group: int) -> bool:
    return K % 64 == 0 and group >= 64 and group % 64 == 0 and K % group == 0


class _W4Method:
    """Shared tail of the two checkpoint formats: keep the packed form when the kernels take it."""

    def _finish(self, layer, q, scale_kn, zero_gn, group, contiguous_groups: bool, dense_fallback, dev=None):
        """``q [K, N]`` ints, ``scale_kn [K / g, N]``, ``zero_gn [K / g, N]`` (values), all on the CPU."""
        dev = layer.scales.device if dev is None else dev
        K = q.shape[0]
        if contiguous_groups and packed_ok(K, group) and scale_kn.dtype in (torch.bfloat16, torch.float16):
            layer.w4_packed = pack_w4(q.T.contiguous()).to(dev)
            layer.w4_scale = scale_kn.T.contiguous().to(dev)
            layer.w4_zero = zero_gn.T.to(scale_kn.dtype).contiguous().to(dev)
            layer.w4_group = group
            layer.weight = None
        else:
            layer.weight = torch.nn.Parameter(dense_fallback().T.contiguous().to(dev), requires_grad=False)
        layer.qweight = layer.qzeros = None

    def apply(self, layer, x):
        if getattr(layer, "weight", None) is not None:
            return ops.linear(x, layer.weight, layer.bias)
        return ops.w4_linear(x, layer.w4_packed, layer.w4_scale, layer.w4_zero, layer.w4_group, layer.bias)


class AWQLinearMethod(_W4Method):
    name = "awq"

    def __init__(self, group_size: int = 128, bits: int = 4):
        self.group_size, self.bits = group_size, bits

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        g = self.group_size if self.group_size > 0 else in_local
        self._g = g
        layer.qweight = param(in_local, out_local // 8, dtype=torch.int32, device=device)
        layer.qzeros = param(in_local // g, out_local // 8, dtype=torch.int32, device=device)
        layer.scales = param(in_local // g, out_local, dtype=dtype, device=device)
        layer.weight = None

    def aux_params(self):
        return {}

    def kn_params(self):
        """Input-major checkpoint tensors ``[K / k_div, N / n_div]`` (how the parallel layers shard them)."""
        g = self._g
        return {"qweight": (1, 8), "qzeros": (g, 8), "scales": (g, 1)}

    def process_weights_after_loading(self, layer):
        if layer.qweight is None:
            return
        qw, sc, qz = layer.qweight.data.cpu(), layer.scales.data.cpu(), layer.qzeros.data.cpu()
        g = self.group_size if self.group_size > 0 else qw.shape[0]
        shifts = torch.tensor([4 * i for i in rb.AWQ_ORDER], dtype=torch.int32)
        q = ((qw.unsqueeze(-1) >> shifts) & 0xF).reshape(qw.shape[0], -1)          # [K, N]
        z = ((qz.unsqueeze(-1) >> shifts) & 0xF).reshape(qz.shape[0], -1)          # [K / g, N]
        self._finish(layer, q, sc, z, g, True, lambda: rb.awq_dequantize(qw, sc, qz, g))


class GPTQLinearMethod(_W4Method):
    name = "gptq"

    def __init__(self, group_size: int = 128, bits: int = 4, desc_act: bool = False):
        self.group_size, self.bits, self.desc_act = group_size, bits, desc_act

    def kn_params(self):
        pack = 32 // self.bits
        return {"qweight": (pack, 1), "qzeros": (self._g, pack), "scales": (self._g, 1), "g_idx": (1, None)}

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        pack = 32 // self.bits
        g = self.group_size if self.group_size > 0 else in_local
        self._g = g
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
        qw, sc, qz, gi = (layer.qweight.data.cpu(), layer.scales.data.cpu(), layer.qzeros.data.cpu(),
                          layer.g_idx.data.cpu())
        K = qw.shape[0] * (32 // self.bits)
        g = self.group_size if self.group_size > 0 else K
        dense = lambda: rb.gptq_dequantize(qw, sc, qz, gi, self.bits)  # noqa: E731
        in_order = bool((gi.long() == torch.arange(K) // g).all())
        if self.bits != 4:
            return self._finish(layer, torch.zeros(K, 0, dtype=torch.int32), sc, sc, g, False, dense)
        shifts = torch.arange(0, 32, 4, dtype=torch.int32)
        q = ((qw.unsqueeze(1) >> shifts.view(1, -1, 1)) & 0xF).reshape(-1, qw.shape[1])          # [K, N]
        z = ((qz.unsqueeze(-1) >> shifts) & 0xF).reshape(qz.shape[0], -1) + 1                    # [K / g, N]
        self._finish(layer, q, sc, z, g, in_order, dense)


class CompressedTensorsW4A16LinearMethod(_W4Method):
    """compressed-tensors ``pack-quantized`` int4 weights with 16-bit activations (W4A16; the reference lists the
    format in ``docs/source/user_guide/feature_guide/quantization.md:4-44``): ``weight_packed [N, K / 8]`` int32
    (eight values per word along k, value ``i`` in bits ``4 i``), ``weight_scale [N, K / g]``, and for asymmetric
    checkpoints ``weight_zero_point [N / 8, K / g]`` int32 (packed along n); symmetric values are stored with an
    offset of 8.  Output-major tensors: the parallel layers shard them like an ordinary weight."""
    name = "w4a16"

    def __init__(self, group_size: int = 128, bits: int = 4, symmetric: bool = True):
        self.group_size, self.bits, self.symmetric = group_size, bits, symmetric

    def create_weights(self, layer, out_local: int, in_local: int, dtype, device):
        g = self.group_size if self.group_size > 0 else in_local
        self._g = g
        layer.weight_packed = param(out_local, in_local // 8, dtype=torch.int32, device=device)
        layer.weight_scale = param(out_local, in_local // g, dtype=dtype, device=device)
        layer.weight_zero_point = None if self.symmetric else param(out_local // 8, in_local // g, dtype=torch.int32,
                                                                    device=device)
        layer.weight = None

    def aux_params(self):
        """(row divisor, column divisor) of the tensors that are smaller than the weight."""
        return {"weight_packed": (1, 8), "weight_scale": (1, self._g), "weight_zero_point": (8, self._g)}

    def process_weights_after_loading(self, layer):
        if layer.weight_packed is None:
            return
        dev = layer.weight_scale.device
        wp, sc = layer.weight_packed.data.cpu(), layer.weight_scale.data.cpu()
        shifts = torch.arange(0, 32, 4, dtype=torch.int32)
        q = ((wp.unsqueeze(-1) >> shifts) & 0xF).reshape(wp.shape[0], -1)                      # [N, K]
        if layer.weight_zero_point is None:
            z = torch.full(sc.shape, 8, dtype=torch.int32)
        else:
            zp = layer.weight_zero_point.data.cpu()                                              # [N / 8, K / g]
            z = ((zp.unsqueeze(1) >> shifts.view(1, -1, 1)) & 0xF).reshape(-1, zp.shape[1])      # [N, K / g]
        g = self._g
        dense = lambda: ((q - z.repeat_interleave(g, 1)).float() * sc.float().repeat_interleave(g, 1)).to(sc.dtype).T  # noqa: E731
        self._finish(layer, q.T.contiguous(), sc.T.contiguous(), z.T.contiguous(), g, True, dense, dev)
        layer.weight_packed = layer.weight_zero_point = layer.weight_scale = None
