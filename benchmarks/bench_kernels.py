"""Kernel micro-benchmarks with roofline fractions (CUDA events, L2 flushed between iterations).

    python benchmarks/bench_kernels.py [--what gemm,attn,elementwise] [--iters 20]

Prints one JSON line per case: achieved GB/s or TFLOP/s and the fraction of the measured peak
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s / 1.59 PFLOP/s).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timeit(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(iters):
    from vllm_kunlun_b200.ops.gemm_cuda import check_status, gemm_bf16
    hbm, tf, src = peaks()
    shapes = [(16, 6144, 4096), (16, 4096, 4096), (16, 28672, 4096), (16, 4096, 14336), (16, 128256, 4096),
              (32, 28672, 4096), (64, 28672, 4096), (128, 28672, 4096), (256, 28672, 4096),
              (2048, 6144, 4096), (8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336)]
    for T, N, K in shapes:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: gemm_bf16(x, w, out=out), iters)
        ms_lib = timeit(lambda: torch.matmul(x, w.T, out=out), iters)
        check_status()
        byt = (T * K + N * K + T * N) * 2
        fl = 2.0 * T * N * K
        gbs, tfl = byt / ms / 1e6, fl / ms / 1e9
        print(json.dumps({"kernel": "gemm_bf16", "T": T, "N": N, "K": K, "ms": round(ms, 4),
                          "cublas_ms": round(ms_lib, 4), "GBps": round(gbs, 1), "TFLOPs": round(tfl, 1),
                          "frac_hbm": round(gbs / hbm, 3), "frac_tensor": round(tfl / tf, 3), "peaks": src}), flush=True)


def bench_gemm_sweep(iters):
    """Decode-shaped GEMMs over split-K factor and CTAs per SM (tuning aid for the launch heuristic)."""
    from vllm_kunlun_b200.ops.gemm_cuda import check_status, gemm_bf16
    hbm, _, src = peaks()
    for T, N, K in [(16, 6144, 4096), (16, 4096, 4096), (16, 28672, 4096), (16, 4096, 14336), (64, 28672, 4096)]:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        for cps in (1, 2, 3):
            for sp in (0, 1, 2, 3, 4, 5, 6, 8, 12):
                ms = timeit(lambda: gemm_bf16(x, w, out=out, splits=sp, ctas_per_sm=cps), iters)
                byt = (T * K + N * K + T * N) * 2
                print(json.dumps({"kernel": "gemm_sweep", "T": T, "N": N, "K": K, "ctas_per_sm": cps, "splits": sp,
                                  "ms": round(ms, 4), "frac_hbm": round(byt / ms / 1e6 / hbm, 3), "peaks": src}), flush=True)
        check_status()


def profile_case(iters):
    """A handful of launches of the two decode hot kernels on inputs larger than L2, sized for an
    ``ncu --set full`` capture (weights 235 MB, KV cache 200 MB)."""
    from vllm_kunlun_b200.ops.attention_cuda import AttnWorkspace, paged_attention_cuda
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_bf16
    x = torch.randn(16, 4096, device="cuda").bfloat16()
    w = (torch.randn(28672, 4096, device="cuda") * 0.02).bfloat16()
    out = torch.empty(16, 28672, device="cuda", dtype=torch.bfloat16)
    xl = torch.randn(4096, 4096, device="cuda").bfloat16()
    wl = (torch.randn(6144, 4096, device="cuda") * 0.02).bfloat16()
    outl = torch.empty(4096, 6144, device="cuda", dtype=torch.bfloat16)
    B, L, Hq, Hkv, D, bs = 16, 3072, 32, 8, 128, 64
    cache = (torch.randn(B * (L // bs) + 1, 2, Hkv, bs, D, device="cuda") * 0.5).bfloat16()
    bt = torch.arange(B * (L // bs), device="cuda", dtype=torch.int32).reshape(B, -1)
    sl = torch.full((B,), L, device="cuda", dtype=torch.int32)
    qsl = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    ws = AttnWorkspace(B, Hq, D, 16, "cuda")
    for _ in range(max(1, iters)):
        gemm_bf16(x, w, out=out)
        gemm_bf16(xl, wl, out=outl)
        paged_attention_cuda(o, q, cache, bt, sl, qsl, D ** -0.5, 1, L, workspace=ws)
    torch.cuda.synchronize()
    print("profile_case done")


def bench_attn(iters):
    from vllm_kunlun_b200.ops.attention_cuda import AttnWorkspace, paged_attention_cuda
    hbm, tf, src = peaks()
    Hq, Hkv, D, bs = 32, 8, 128, 64
    for B, L in [(16, 2048), (16, 3072), (16, 4096), (64, 2048), (1, 8192)]:
        nblk = B * (L // bs) + 1
        cache = (torch.randn(nblk, 2, Hkv, bs, D, device="cuda") * 0.5).bfloat16()
        bt = torch.arange(B * (L // bs), device="cuda", dtype=torch.int32).reshape(B, -1)
        sl = torch.full((B,), L, device="cuda", dtype=torch.int32)
        qsl = torch.arange(B + 1, device="cuda", dtype=torch.int32)
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        out = torch.empty_like(q)
        ws = AttnWorkspace(B, Hq, D, 32, "cuda")
        for splits in (None, 1, 4, 8, 16):
            ms = timeit(lambda: paged_attention_cuda(out, q, cache, bt, sl, qsl, D ** -0.5, 1, L, workspace=ws,
                                                     num_splits=splits), iters)
            byt = B * L * Hkv * D * 2 * 2
            print(json.dumps({"kernel": "paged_attention_decode", "B": B, "L": L, "splits": splits, "ms": round(ms, 4),
                              "GBps": round(byt / ms / 1e6, 1), "frac_hbm": round(byt / ms / 1e6 / hbm, 3),
                              "peaks": src}), flush=True)
    # prefill
    for B, L in [(1, 2048), (4, 2048), (2, 8192)]:
        nblk = B * (L // bs) + 1
        cache = (torch.randn(nblk, 2, Hkv, bs, D, device="cuda") * 0.5).bfloat16()
        bt = torch.arange(B * (L // bs), device="cuda", dtype=torch.int32).reshape(B, -1)
        sl = torch.full((B,), L, device="cuda", dtype=torch.int32)
        qsl = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * L)
        q = torch.randn(B * L, Hq, D, device="cuda").bfloat16()
        out = torch.empty_like(q)
        ms = timeit(lambda: paged_attention_cuda(out, q, cache, bt, sl, qsl, D ** -0.5, L, L), max(3, iters // 4))
        fl = 4.0 * B * Hq * D * L * L / 2
        print(json.dumps({"kernel": "paged_attention_prefill", "B": B, "L": L, "ms": round(ms, 4),
                          "TFLOPs": round(fl / ms / 1e9, 1), "frac_tensor": round(fl / ms / 1e9 / tf, 3),
                          "peaks": src}), flush=True)


def bench_elementwise(iters):
    from vllm_kunlun_b200 import ops
    hbm, _, src = peaks()
    for T in (16, 8192):
        H = 4096
        x = torch.randn(T, H, device="cuda").bfloat16()
        r = torch.randn(T, H, device="cuda").bfloat16()
        w = torch.ones(H, device="cuda").bfloat16()
        ms = timeit(lambda: ops.add_rmsnorm(x, r, w, 1e-5), iters)
        print(json.dumps({"kernel": "add_rmsnorm", "T": T, "H": H, "ms": round(ms, 4),
                          "GBps": round(T * H * 2 * 4 / ms / 1e6, 1), "frac_hbm": round(T * H * 8 / ms / 1e6 / hbm, 3)}))
        gu = torch.randn(T, 2 * 14336, device="cuda").bfloat16()
        ms = timeit(lambda: ops.silu_and_mul(gu), iters)
        print(json.dumps({"kernel": "silu_and_mul", "T": T, "ms": round(ms, 4),
                          "GBps": round(T * 14336 * 2 * 3 / ms / 1e6, 1),
                          "frac_hbm": round(T * 14336 * 6 / ms / 1e6 / hbm, 3)}), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn,elementwise")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    for w in a.what.split(","):
        {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "gemm_sweep": bench_gemm_sweep, "profile_case": profile_case}[w](a.iters)
