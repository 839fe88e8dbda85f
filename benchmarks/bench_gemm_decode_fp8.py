"""Decode-sized fp8 block-scaled linears: the cluster split-K kernel (csrc/gemm/gemm_decode.cu, fp8 template)
against the grouped block-scaled kernel (csrc/gemm/gemm_grouped.cu), each timed in a CUDA-graph chain of
``--layers`` launches over distinct weights, with and without the activation quantiser in front.

    python benchmarks/bench_gemm_decode_fp8.py

Prints microseconds per launch next to weight bytes / measured HBM bandwidth.
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
ap.add_argument("--hbm-gbs", type=float, default=6548.5)
ap.add_argument("--splits", type=int, nargs="+", default=[0, 1, 2, 4, 8])
ap.add_argument("--shapes", type=str, default="2048x4096,4096x2048,5120x2048,2048x4096,7168x2048,1536x7168")
a = ap.parse_args()
dev, L = "cuda", a.layers
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
        ws = [torch.randint(0, 120, (N, K), device=dev, dtype=torch.uint8) for _ in range(L)]
        sc = [torch.rand((N + 127) // 128, (K + 127) // 128, device=dev) * 0.01 + 0.001 for _ in range(L)]
        sc3 = [s.unsqueeze(0).contiguous() for s in sc]
        for B in a.batch:
            x = torch.randn(B, K, device=dev).bfloat16()
            xq, st = C.quant_fp8_group(x, False, None, 4)
            out = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
            ideal = N * K / (a.hbm_gbs * 1e3)
            cells = []
            for S in a.splits:
                if S > (8 if B <= 16 else 4):
                    continue
                try:
                    t = graph_time(lambda: [C.gemm_decode_fp8(out, xq, w, None, st, s, S) for w, s in zip(ws, sc)])
                    cells.append(f"S={S}: {t:.2f}")
                except RuntimeError:
                    cells.append(f"S={S}: err")
            t = graph_time(lambda: [C.grouped_gemm(out, xq, w, None, None, st, s, 0) for w, s in zip(ws, sc3)])
            cells.append(f"grouped: {t:.2f}")

            def with_quant():
                for w, s in zip(ws, sc):
                    q2, s2 = C.quant_fp8_group(x, False, None, 4)
                    C.gemm_decode_fp8(out, q2, w, None, s2, s, 0)
            cells.append(f"quant+S=0: {graph_time(with_quant):.2f}")
            print(f"fp8 {B}x{N}x{K} ideal {ideal:.2f} | " + " | ".join(cells), flush=True)
        del ws
check_status()
