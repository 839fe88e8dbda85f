"""Device timings of the sampling, gated-delta-net, conv, LoRA and MTP-glue kernels (CUDA events, L2 flushed
between iterations, 3 warm-ups), reported against the algorithmic bytes and the measured copy bandwidth.

    python benchmarks/bench_misc_kernels.py [--case sample|gdn|conv|lora|all] [--small]

``--small`` shrinks every case to a few hundred MB so that a profiler capture of one launch ends quickly."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_kunlun_b200 import ops  # noqa: E402

PEAK_GBS = 6548.5
try:
    with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
        PEAK_GBS = float(json.load(f).get("hbm_gbs", PEAK_GBS))
except Exception:  # noqa: BLE001
    pass


def timeit(fn, iters=10, warm=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def report(name, sec, nbytes, extra=""):
    gbs = nbytes / sec / 1e9
    print(json.dumps({"kernel": name, "us": round(sec * 1e6, 1), "GB/s": round(gbs, 1),
                      "frac_of_measured_copy_bw": round(gbs / PEAK_GBS, 3), "note": extra}))


def case_sample(small):
    B, V = (16, 151936) if not small else (16, 32000)
    logits = torch.randn(B, V, device="cuda").to(torch.bfloat16)
    t = torch.full((B,), 0.8, device="cuda")
    k = torch.full((B,), 50, dtype=torch.int32, device="cuda")
    p = torch.full((B,), 0.9, device="cuda")
    sec = timeit(lambda: ops.topk_topp_sample(logits, t, k, p, seed=1))
    report("topk_topp_sample_kernel", sec, B * V * 2, f"B={B} V={V}; 11 passes over the row, L2 resident after the first")
    g = torch.zeros(B, device="cuda")
    sec = timeit(lambda: ops.topk_topp_sample(logits, g, None, None))
    report("topk_topp_sample_kernel(greedy)", sec, B * V * 2, f"B={B} V={V}")

    def torch_path():
        lg = logits.float() / 0.8
        from vllm_kunlun_b200.ops.reference import misc as ref
        lg = ref.apply_top_k_top_p(lg, k.long(), p)
        pr = lg.softmax(-1)
        return (pr / torch.empty_like(pr).exponential_()).argmax(-1)
    sec = timeit(torch_path)
    report("sort-based torch sampler (comparison)", sec, B * V * 2)


def case_gdn(small):
    Hk, Hv, D = 16, 32, 128
    for name, R, L in (("decode", 16, 1), ("prefill", 16 if not small else 4, 2048 if not small else 512)):
        T = R * L
        C = 2 * Hk * D + Hv * D
        mixed = torch.randn(T, C, device="cuda").to(torch.bfloat16)
        q, k = mixed[:, :Hk * D].view(T, Hk, D), mixed[:, Hk * D:2 * Hk * D].view(T, Hk, D)
        v = mixed[:, 2 * Hk * D:].view(T, Hv, D)
        g = -torch.rand(T, Hv, device="cuda")
        beta = torch.rand(T, Hv, device="cuda")
        states = torch.zeros(R, Hv, D, D, device="cuda")
        cu = (torch.arange(R + 1, device="cuda") * L).int()
        idx = torch.arange(R, device="cuda").int()
        init = torch.ones(R, device="cuda").int()
        sec = timeit(lambda: ops.gated_delta_rule(q, k, v, g, beta, states, cu, idx, init))
        nbytes = 2 * states.numel() * 4 + T * C * 2 + T * Hv * D * 2
        report(f"gdn_recurrent_kernel({name})", sec, nbytes, f"R={R} L={L}; {T * Hv * 3 * D * D * 2 / sec / 1e12:.2f} TFLOP/s fp32 FMA")


def case_conv(small):
    C, W = 8192, 4
    T = 32768 if not small else 4096
    x = torch.randn(T, C, device="cuda").to(torch.bfloat16)
    w = torch.randn(C, W, device="cuda").to(torch.bfloat16)
    R = 16
    cu = (torch.arange(R + 1, device="cuda") * (T // R)).int()
    states = torch.zeros(R, W - 1, C, device="cuda", dtype=torch.bfloat16)
    idx = torch.arange(R, device="cuda").int()
    init = torch.zeros(R, device="cuda").int()
    sec = timeit(lambda: ops.causal_conv1d_fn(x, w, None, cu, states, idx, init, True))
    report("conv1d_fwd_kernel + conv1d_state_kernel", sec, 2 * T * C * 2, f"T={T} C={C}")
    xb = torch.randn(16, C, device="cuda").to(torch.bfloat16)
    sec = timeit(lambda: ops.causal_conv1d_update(xb, states, w, None, idx, True))
    report("conv1d_update_kernel", sec, 2 * 16 * C * 2 + 2 * states.numel() * 2, "B=16")


def case_lora(small):
    K, N, r, L = 4096, 6144, 16, 4
    T = 8192 if not small else 1024
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    A = torch.randn(L, r, K, device="cuda").to(torch.bfloat16)
    Bm = torch.randn(L, N, r, device="cuda").to(torch.bfloat16)
    out = torch.zeros(T, N, device="cuda", dtype=torch.bfloat16)
    # prefill: runs of 512 tokens per adapter; decode-like: an adapter drawn per token
    patterns = (("segments of 512", (torch.arange(T, device="cuda") // 512 % L).int()),
                ("adapter per token", torch.randint(0, L, (T,), device="cuda", dtype=torch.int32)))
    for name, ids in patterns:
        sec = timeit(lambda: ops.lora_shrink(x, A, ids, 1.0))
        report("lora_shrink_kernel", sec, T * K * 2 + T * r * 4, f"T={T} K={K} r={r}, {name}")
        h = ops.lora_shrink(x, A, ids, 1.0)
        sec = timeit(lambda: ops.lora_expand(h, Bm, ids, out, 0, True))
        report("lora_expand_kernel", sec, 2 * T * N * 2 + T * r * 4, f"T={T} N={N} r={r}, {name}")


def case_gemm_splits(small):
    """Decode-sized bf16 GEMMs of an 8B dense model at TP 1-8: default K split against forced 1-8 equal parts."""
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_bf16
    shapes = [("qkv tp8", 768, 4096), ("qkv tp4", 1536, 4096), ("qkv tp2", 3072, 4096), ("qkv tp1", 6144, 4096),
              ("o tp1", 4096, 4096), ("o tp2", 4096, 2048), ("o tp4", 4096, 1024), ("down tp1", 4096, 14336),
              ("down tp2", 4096, 7168), ("down tp4", 4096, 3584), ("down tp8", 4096, 1792),
              ("gate_up tp8", 3584, 4096)]
    for name, N, K in shapes[:3] if small else shapes:
        x = torch.randn(16, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        out = torch.empty(16, N, device="cuda", dtype=torch.bfloat16)
        res = {"default": timeit(lambda: gemm_bf16(x, w, None, out), iters=15, warm=4)}
        for sp in (1, 2, 3, 4, 6, 8):
            res[str(sp)] = timeit(lambda: gemm_bf16(x, w, None, out, splits=sp), iters=15, warm=4)
        print(json.dumps({"kernel": "gemm_bf16", "shape": f"16x{N}x{K}", "name": name, "tiles": (N + 127) // 128,
                          "us_by_splits": {k: round(v * 1e6, 1) for k, v in res.items()}}))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    cases = {"sample": case_sample, "gdn": case_gdn, "conv": case_conv, "lora": case_lora}
    explicit = {"gemm_splits": case_gemm_splits}  # not part of "all"
    with torch.inference_mode():
        for n, fn in cases.items():
            if a.case in ("all", n):
                fn(a.small)
        if a.case in explicit:
            explicit[a.case](a.small)
