"""Decode-sized GEMM shapes of a Qwen3-30B-A3B layer (16 tokens, 128 experts, top-8): fp8 dense projections, the two
grouped fp8 expert GEMMs and the whole fused MoE block.  CUDA events, 256 MB L2 flush between iterations, 3 warm-ups,
median of 10; "ideal" = weight bytes over the measured copy bandwidth.

    python benchmarks/bench_moe_decode_shapes.py
"""
import os, sys, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_kunlun_b200 import ops
from vllm_kunlun_b200.ops import _ext
from vllm_kunlun_b200.models.moe import _quant_block_device
C = _ext.C()
dev = "cuda"
flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
def timeit(fn, it=10):
    for _ in range(3): fn()
    torch.cuda.synchronize(); ts = []
    for _ in range(it):
        flush.fill_(1); e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); torch.cuda.synchronize(); ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort(); return ts[len(ts) // 2]
torch.manual_seed(0)
T, H, I, E, k = 16, 2048, 768, 128, 8
x = torch.randn(T, H, device=dev).bfloat16()
for name, N, K in (("qkv", 5120, 2048), ("o_proj", 2048, 4096)):
    w, s = _quant_block_device(torch.randn(N, K, device=dev) * 0.05)
    xin = torch.randn(T, K, device=dev).bfloat16()
    q, st = C.quant_fp8_group(xin, False, None, 4)
    out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    us = timeit(lambda: C.grouped_gemm(out, q, w.view(torch.uint8), None, None, st, s.unsqueeze(0).contiguous(), 0))
    print(f"{name} fp8 dense {T}x{N}x{K}: {us:.1f} us, ideal {N*K/6.55e6:.1f} us")
    wb = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    us = timeit(lambda: ops.linear(xin, wb))
    print(f"{name} bf16 dense: {us:.1f} us, ideal {2*N*K/6.55e6:.1f} us")
w13 = torch.stack([_quant_block_device(torch.randn(2 * I, H, device=dev) * 0.05)[0] for _ in range(E)])
s13 = torch.stack([_quant_block_device(torch.randn(2 * I, H, device=dev) * 0.05)[1] for _ in range(E)])
w2 = torch.stack([_quant_block_device(torch.randn(H, I, device=dev) * 0.05)[0] for _ in range(E)])
s2 = torch.stack([_quant_block_device(torch.randn(H, I, device=dev) * 0.05)[1] for _ in range(E)])
wts, ids = ops.moe_route(torch.randn(T, E, device=dev), k, "softmax", True)
xs, pos, lod, st = C.moe_prepare_small(x, ids.contiguous(), None, E, E, True)
used = int((lod[1:] - lod[:-1] > 0).sum())
M = xs.shape[0]
h = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=dev)
us = timeit(lambda: C.grouped_gemm(h, xs, w13.view(torch.uint8), lod, None, st, s13, 0))
print(f"w13 grouped fp8 ({used} experts used): {us:.1f} us, ideal {used*2*I*H/6.55e6:.1f} us")
q2, st2 = C.act_mul_quant_fp8(h, 0, lod[E:])
y = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
us = timeit(lambda: C.grouped_gemm(y, q2, w2.view(torch.uint8), lod, None, st2, s2, 0))
print(f"w2 grouped fp8: {us:.1f} us, ideal {used*I*H/6.55e6:.1f} us")
us = timeit(lambda: ops.fused_moe(x, w13, w2, wts, ids, "silu", None, None, s13, s2, (128, 128), None))
print(f"whole fused_moe: {us:.1f} us")
