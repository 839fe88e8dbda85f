"""Cluster size / residency sweep of the decode GEMM (csrc/gemm/gemm_decode.cu), timed in a CUDA-graph chain of
``--layers`` launches over distinct weights (cold weights, queued launches - as inside a decode step).

    python benchmarks/bench_gemm_decode_sweep.py --tp 1 8

Prints microseconds per launch for every (cluster size S, CTAs per SM) pair next to bytes / measured HBM bandwidth.
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
ap.add_argument("--tp", type=int, nargs="+", default=[1, 8])
ap.add_argument("--layers", type=int, default=32)
ap.add_argument("--batch", type=int, default=16)
ap.add_argument("--iters", type=int, default=10)
ap.add_argument("--hbm-gbs", type=float, default=6548.5)
ap.add_argument("--splits", type=int, nargs="+", default=[0, 1, 2, 4, 8])
ap.add_argument("--cps", type=int, nargs="+", default=[1, 2])
ap.add_argument("--stages", type=int, nargs="+", default=[0])
a = ap.parse_args()
dev, dt, L, B = "cuda", torch.bfloat16, a.layers, a.batch
C = _ext.C()


def chain_time(ws, x, out, S, cps, act, stages):
    def run():
        for w in ws:
            C.gemm_decode(out, x, w, None, S, stages, cps, act)
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
        ts.append(e0.elapsed_time(e1) * 1e3 / len(ws))
    return statistics.median(ts)


with torch.inference_mode():
    for tp in a.tp:
        hq, hkv, inter, H = 32 // tp, max(1, 8 // tp), 14336 // tp, 4096
        shapes = [("qkv", (hq + 2 * hkv) * 128, H, 0), ("o", H, hq * 128, 0), ("gate_up", 2 * inter, H, 1),
                  ("down", H, inter, 0)]
        for name, N, K, act in shapes:
            ws = [(torch.randn(N, K, device=dev) * 0.02).to(dt) for _ in range(L)]
            x = torch.randn(B, K, device=dev).to(dt)
            out = torch.empty(B, N // 2 if act else N, device=dev, dtype=dt)
            ideal = N * K * 2 / (a.hbm_gbs * 1e3)
            cells = []
            for S in a.splits:
                for cps in a.cps:
                    for st in a.stages:
                        try:
                            t = chain_time(ws, x, out, S, cps, act, st)
                            cells.append(f"S={S} cps={cps}" + (f" st={st}" if st else "") + f": {t:.2f}")
                        except RuntimeError as e:
                            cells.append(f"S={S} cps={cps}: err")
            print(f"tp{tp} {name} {B}x{N}x{K} ideal {ideal:.2f} | " + " | ".join(cells), flush=True)
            del ws
check_status()
