"""Quantised linear methods on the CPU oracle path: int8 W8A8, AWQ and GPTQ int4, fp8 block-128 with TP sharding."""
import pytest
import torch

from vllm_kunlun_b200.models.layers import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from vllm_kunlun_b200.ops.reference import basic as rb


def test_int8_w8a8_linear_dynamic_and_static():
    torch.manual_seed(0)
    w = torch.randn(48, 64) * 0.1
    x = torch.randn(5, 64)
    lin = ReplicatedLinear(64, 48, dtype=torch.float32, device="cpu", quant="int8")
    lin.method.quantize_(lin, w)
    torch.testing.assert_close(lin(x), x @ w.T, atol=0.05, rtol=0.05)
    stat = ReplicatedLinear(64, 48, dtype=torch.float32, device="cpu", quant="int8", quant_kw={"static_input_scale": True})
    stat.method.quantize_(stat, w)
    stat.input_scale.data.fill_(float(x.abs().max()) / 127)
    torch.testing.assert_close(stat(x), x @ w.T, atol=0.08, rtol=0.08)


def test_awq_linear_unpacks_once_and_matches_dequantised_weight():
    torch.manual_seed(1)
    K, N, g = 128, 64, 32
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(0, 16, (K // g, N))
    sc = torch.rand(K // g, N) * 0.05
    lin = ReplicatedLinear(K, N, dtype=torch.float32, device="cpu", quant="awq", quant_kw={"group_size": g})
    lin.qweight.data.copy_(rb.awq_pack(wi))
    lin.qzeros.data.copy_(rb.awq_pack(zi))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    assert lin.qweight is None and lin.weight.shape == (N, K)
    dense = ((wi - zi.repeat_interleave(g, 0)).float() * sc.repeat_interleave(g, 0))  # [K, N]
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ dense, atol=1e-4, rtol=1e-4)


def test_gptq_linear_matches_dequantised_weight():
    torch.manual_seed(2)
    K, N, g = 128, 32, 64
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(1, 16, (K // g, N))  # stored minus one
    sc = torch.rand(K // g, N) * 0.05
    qw = torch.zeros(K // 8, N, dtype=torch.int64)
    for j in range(8):
        qw |= wi[j::8].long() << (4 * j)
    qz = torch.zeros(K // g, N // 8, dtype=torch.int64)
    for j in range(8):
        qz |= (zi[:, j::8].long() - 1) << (4 * j)
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    lin = ReplicatedLinear(K, N, dtype=torch.float32, device="cpu", quant="gptq", quant_kw={"group_size": g})
    lin.qweight.data.copy_(to32(qw))
    lin.qzeros.data.copy_(to32(qz))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    dense = (wi - zi.repeat_interleave(g, 0)).float() * sc.repeat_interleave(g, 0)
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ dense, atol=1e-4, rtol=1e-4)


def test_fp8_block_scales_shard_with_the_weight():
    """Row shards of a merged projection and column shards of a row-parallel layer take the matching scale blocks
    (ceil-division rule for partitions that are not multiples of 128)."""
    torch.manual_seed(3)
    K = 256
    parts = [256, 128]
    w = torch.randn(sum(parts), K) * 0.1
    q, s = rb.quant_fp8_block(w, (128, 128))
    deq = rb.dequant_fp8_block(q, s, (128, 128))
    x = torch.randn(4, K)
    outs = []
    for rank in range(2):
        lin = ColumnParallelLinear(K, parts, dtype=torch.float32, device="cpu", quant="fp8", tp_size=2, tp_rank=rank)
        off_w, off_s = 0, 0
        for i, n in enumerate(parts):
            lin.load("weight", q[off_w:off_w + n], i)
            lin.load("weight_scale_inv", s[off_s:off_s + n // 128], i)
            off_w, off_s = off_w + n, off_s + n // 128
        outs.append(lin(x))
    full = x @ deq.T
    got = torch.cat([outs[0][:, :128], outs[1][:, :128], outs[0][:, 128:], outs[1][:, 128:]], -1)
    torch.testing.assert_close(got, full, atol=0.2, rtol=0.1)
    row = [RowParallelLinear(K, 64, dtype=torch.float32, device="cpu", quant="fp8", tp_size=2, tp_rank=r, reduce_results=False)
           for r in range(2)]
    w2 = torch.randn(64, K) * 0.1
    q2, s2 = rb.quant_fp8_block(w2, (128, 128))
    acc = 0
    for r, lin in enumerate(row):
        lin.load("weight", q2)
        lin.load("weight_scale_inv", s2)
        acc = acc + lin(x[:, r * 128:(r + 1) * 128])
    torch.testing.assert_close(acc, x @ rb.dequant_fp8_block(q2, s2, (128, 128)).T, atol=0.2, rtol=0.1)


def test_w4_pack_roundtrip_and_pair_extraction_order():
    """The kernels' packed layout: unpack inverts pack, and the pair (2 j, 2 j + 1) of a word's eight k values is
    `(w >> 4 j) & 0x000F000F` (low half, high half) - the extraction the decode GEMM performs."""
    from vllm_kunlun_b200.quantization.int4 import pack_w4, unpack_w4
    torch.manual_seed(4)
    q = torch.randint(0, 16, (5, 64))
    packed = pack_w4(q)
    assert packed.shape == (5, 32) and packed.dtype == torch.uint8
    assert torch.equal(unpack_w4(packed), q.to(torch.int32))
    b = packed.view(5, 8, 4).long()
    words = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    for j in range(4):
        t = (words >> (4 * j)) & 0x000F000F
        assert torch.equal(t & 0xFFFF, q.view(5, 8, 8)[..., 2 * j].long())
        assert torch.equal(t >> 16, q.view(5, 8, 8)[..., 2 * j + 1].long())


@pytest.mark.parametrize("fmt,g", [("awq", 128), ("awq", 64), ("gptq", 128)])
def test_w4_linear_keeps_packed_weights(fmt, g):
    """bf16 AWQ / GPTQ layers with kernel-friendly shapes keep only the packed bytes (+ scale / zero per group) and
    give the result of the de-quantised weight; a GPTQ layer with a permuted g_idx falls back to a 16-bit weight."""
    torch.manual_seed(5)
    K, N = 256, 48 if fmt == "gptq" else 64
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(1, 16, (K // g, N))
    sc = (torch.rand(K // g, N) * 0.05 + 0.01).bfloat16()
    lin = ReplicatedLinear(K, N, dtype=torch.bfloat16, device="cpu", quant=fmt, quant_kw={"group_size": g})
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    if fmt == "awq":
        lin.qweight.data.copy_(rb.awq_pack(wi))
        lin.qzeros.data.copy_(rb.awq_pack(zi))
    else:
        qw = torch.zeros(K // 8, N, dtype=torch.int64)
        for j in range(8):
            qw |= wi[j::8].long() << (4 * j)
        qz = torch.zeros(K // g, N // 8, dtype=torch.int64)
        for j in range(8):
            qz |= (zi[:, j::8].long() - 1) << (4 * j)
        lin.qweight.data.copy_(to32(qw))
        lin.qzeros.data.copy_(to32(qz))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    assert lin.weight is None and lin.w4_packed.shape == (N, K // 2) and lin.w4_scale.shape == (N, K // g)
    dense = ((wi - zi.repeat_interleave(g, 0)).float() * sc.float().repeat_interleave(g, 0)).bfloat16()   # [K, N]
    x = torch.randn(3, K).bfloat16()
    torch.testing.assert_close(lin(x).float(), (x.float() @ dense.float()).bfloat16().float(), atol=2e-2, rtol=2e-2)
    if fmt == "gptq":
        lin2 = ReplicatedLinear(K, N, dtype=torch.bfloat16, device="cpu", quant="gptq", quant_kw={"group_size": g})
        lin2.qweight.data.copy_(to32(qw)); lin2.qzeros.data.copy_(to32(qz)); lin2.scales.data.copy_(sc)
        lin2.g_idx.data.copy_(torch.arange(K, dtype=torch.int32).flip(0) // g)       # activation-order checkpoint
        lin2.method.process_weights_after_loading(lin2)
        assert lin2.weight is not None and lin2.weight.shape == (N, K)
