"""Decode-sized linears over 4-bit weights: the decode GEMM that streams the packed bytes and de-quantises in the
kernel (csrc/gemm/gemm_decode.cu, 4-bit path) against the same kernel over a 16-bit copy of the weight, each timed in
a CUDA-graph chain of ``--layers`` launches over distinct weights (cold weights, queued launches, as in a decode step).

    python benchmarks/bench_gemm_decode_w4.py

Prints microseconds per launch next to packed weight bytes / measured HBM bandwidth.
"""
import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200.ops import _ext  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--layers", type=int, default=32)
ap.add_argument("--batch", type=int, nargs="+", default=[16, 32])
ap.add_argument("--iters", type=int, default=10)
ap.add_argument("--group", type=int, default=128)
ap.add_argument("--hbm-gbs", type=float, default=6548.5)
ap.add_argument("--splits", type=int, nargs="+", default=[0, 1, 2, 4, 8])
ap.add_argument("--shapes", type=str, default="6144x4096,4096x4096,28672x4096,4096x14336")
a = ap.parse_args()
dev, L, G = "cuda", a.layers, a.group
C = _ext.C()


def graph_time(run):
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / L)
    return statistics.median(ts)


with torch.inference_mode():
    for shp in a.shapes.split(","):
        N, K = (int(v) for v in shp.split("x"))
        pk = [torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8) for _ in range(L)]
        sc = [(torch.rand(N, K // G, device=dev) * 0.02 + 0.005).bfloat16() for _ in range(L)]
        zr = [torch.randint(0, 16, (N, K // G), device=dev).bfloat16() for _ in range(L)]
        for B in a.batch:
            x = torch.randn(B, K, device=dev).bfloat16()
            out = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
            ideal = (N * K / 2 + N * (K // G) * 4) / (a.hbm_gbs * 1e3)
            cells = []
            for S in a.splits:
                if S > (8 if B <= 16 else 4):
                    continue
                try:
                    t = graph_time(lambda: [C.gemm_decode_w4(out, x, p, s, z, None, G, S, 0) for p, s, z in zip(pk, sc, zr)])
                    cells.append(f"S={S}: {t:.2f}")
                except RuntimeError:
                    cells.append(f"S={S}: err")
            print(f"w4 {B}x{N}x{K} g{G} ideal {ideal:.2f} | " + " | ".join(cells), flush=True)
        del pk
        # the same shapes over 16-bit weights (4x the bytes); fewer layers when the copies would not fit comfortably
        Lw = L if N * K * 2 * L < (24 << 30) else max(4, (24 << 30) // (N * K * 2))
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(Lw)]
        for B in a.batch:
            x = torch.randn(B, K, device=dev).bfloat16()
            out = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
            t = graph_time(lambda: [C.gemm_decode(out, x, w, None, 0, 0, 0, 0) for w in ws]) * L / Lw
            print(f"16-bit {B}x{N}x{K} ideal {N * K * 2 / (a.hbm_gbs * 1e3):.2f} | S=0: {t:.2f}", flush=True)
        del ws
check_status()
