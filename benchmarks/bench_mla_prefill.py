"""MLA prefill: the up-projected 192 / 128 form on tcgen05 (csrc/attention/prefill_umma.cu, MLA instantiation; the
kv_b_proj up-projection of the keys included) against the absorbed 576 / 512 form (the two per-head products around
it included).  CUDA events, 3 warm-ups, median of 10; a 256 MB buffer is written between iterations (L2 flush).

    python benchmarks/bench_mla_prefill.py                     # 4 requests x 2048 new tokens, 16 heads (one TP=8 rank)
    python benchmarks/bench_mla_prefill.py --heads 128 --reqs 2
"""
import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200 import ops  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--reqs", type=int, default=4)
ap.add_argument("--q-len", type=int, default=2048)
ap.add_argument("--heads", type=int, default=16)
ap.add_argument("--bf16-tflops", type=float, default=1590.0, help="measured cuBLAS bf16 burst peak")
a = ap.parse_args()
dev, dt, bs = "cuda", torch.bfloat16, 64
B, QL, N = a.reqs, a.q_len, a.heads
T = B * QL
g = torch.Generator(device=dev).manual_seed(0)
rnd = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.3).to(dt)  # noqa: E731
q_nope, q_pe, kv_c, k_pe = rnd(T, N, 128), rnd(T, N, 64), rnd(T, 512), rnd(T, 64)
w_kvb = rnd(N * 256, 512)
w3 = w_kvb.view(N, 256, 512)
w_uk, w_uv = w3[:, :128].contiguous(), w3[:, 128:].transpose(1, 2).contiguous()
nb = -(-QL // bs)
cache = torch.zeros(B * nb + 1, bs, 576, device=dev, dtype=dt)
bt = (torch.arange(B * nb, device=dev, dtype=torch.int32) + 1).view(B, nb)
slots = torch.cat([(bt[r].long().repeat_interleave(bs) * bs + torch.arange(nb * bs, device=dev) % bs)[:QL] for r in range(B)])
ops.concat_and_cache_mla(kv_c, k_pe, cache, slots)
sl = torch.full((B,), QL, device=dev, dtype=torch.int32)
qsl = torch.arange(0, (B + 1) * QL, QL, device=dev, dtype=torch.int32)
scale = 192 ** -0.5
flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
pairs = B * QL * (QL + 1) // 2          # (query, key) pairs under the causal mask


def up_projected():
    q = torch.cat([q_nope, q_pe], -1)
    kv = ops.linear(kv_c, w_kvb)
    return ops.mla_prefill_attention(q, kv, k_pe, qsl[:-1], sl, qsl, True, scale, QL)[0]


def absorbed():
    qf = torch.cat([ops.bmm_heads(q_nope, w_uk), q_pe], -1)
    o = ops.mla_attention(qf, cache, bt, sl, qsl, scale, 512, QL, QL)
    return ops.bmm_heads(o, w_uv)


def timeit(fn):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(10):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


print(f"# MLA prefill: {B} x {QL} new tokens, {N} heads, causal; attention FLOPs: up-projected "
      f"{2 * pairs * N * 320 / 1e12:.3f} T (+ {2 * T * 512 * N * 256 / 1e12:.3f} T up-projection), absorbed "
      f"{2 * pairs * N * 1088 / 1e12:.3f} T (+ {2 * T * N * 2 * 128 * 512 / 1e12:.3f} T per-head products)")
print("| form | ms | attention TFLOP/s (own FLOPs) | of measured bf16 peak |")
print("|---|---|---|---|")
res = {}
for name, fn, fl in (("up-projected 192 / 128, tcgen05", up_projected, 2 * pairs * N * 320 + 2 * T * 512 * N * 256),
                     ("absorbed 576 / 512", absorbed, 2 * pairs * N * 1088 + 2 * T * N * 2 * 128 * 512)):
    ms = timeit(fn)
    res[name] = fn().float()
    tf = fl / (ms * 1e-3) / 1e12
    print(f"| {name} | {ms:.3f} | {tf:.0f} | {tf / a.bf16_tflops:.2f} |", flush=True)
x, y = res.values()
print(f"max |difference| between the forms: {(x - y).abs().max().item():.4g} (values up to {y.abs().max().item():.3g})")
check_status()
