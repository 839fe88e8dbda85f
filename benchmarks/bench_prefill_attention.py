"""Paged GQA prefill attention: the tcgen05 kernel (csrc/attention/prefill_umma.cu) against the mma.sync kernel
(csrc/attention/paged_attention.cu).  CUDA events, 3 warm-ups, median of 10; a 256 MB buffer is written between
iterations (L2 flush).

    python benchmarks/bench_prefill_attention.py                 # 4 requests x 2048 tokens, 32 q / 8 kv heads
    python benchmarks/bench_prefill_attention.py --reqs 1 --q-len 8192 --ctx 24576   # a chunk at long context
"""
import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200.ops import attention_cuda  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--reqs", type=int, default=4)
ap.add_argument("--q-len", type=int, default=2048)
ap.add_argument("--ctx", type=int, default=0, help="cached tokens in front of the chunk")
ap.add_argument("--heads", type=int, default=32)
ap.add_argument("--kv-heads", type=int, default=8)
ap.add_argument("--trace", action="store_true", help="phase timestamps of the tcgen05 kernel (one launch)")
ap.add_argument("--bf16-tflops", type=float, default=1590.0, help="measured cuBLAS bf16 burst peak")
a = ap.parse_args()
dev, dt, D, bs = "cuda", torch.bfloat16, 128, 64
B, QL, S = a.reqs, a.q_len, a.ctx + a.q_len
nb_per = -(-S // bs)
cache = (torch.randn(B * nb_per + 1, 2, a.kv_heads, bs, D, device=dev) * 0.5).to(dt)
bt = (torch.arange(B * nb_per, device=dev, dtype=torch.int32) + 1).view(B, nb_per)
sl = torch.full((B,), S, device=dev, dtype=torch.int32)
qsl = torch.arange(0, (B + 1) * QL, QL, device=dev, dtype=torch.int32)
q = (torch.randn(B * QL, a.heads, D, device=dev) * 0.5).to(dt)
out = torch.empty_like(q)
flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
# causal: row r of a request sees ctx + r + 1 keys; QK^T and PV
flops = 4.0 * D * a.heads * B * sum(a.ctx + r + 1 for r in range(QL))


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


if a.trace:
    from vllm_kunlun_b200.ops import _ext
    C = _ext.C()
    n_cta = B * a.heads * -(-QL // 128)
    tr = torch.zeros(n_cta * 24, dtype=torch.int64, device=dev)
    for _ in range(2):
        tr.zero_()
        C.set_kernel_trace(tr)
        attention_cuda.paged_attention_cuda(out, q, cache, bt, sl, qsl, D ** -0.5, QL, S)
        torch.cuda.synchronize()
        C.set_kernel_trace(None)
    t = tr.view(-1, 24).cpu()
    t = t[(t[:, 0] > 0) & (t[:, 8] > 0)]
    names = ["start", "first S", "t4 S seen", "t4 max done", "t4 P buffer free", "t4 P written", "loop done", "t5 S seen",
             "t20 S seen", "t4 P seen by issuer", "end", "t4 S in registers", "t3 P.V issued", "t5 S issued"]
    rel = t - t[:, :1]
    print(f"# phase trace over {t.shape[0]} CTAs with > 20 tiles: ns after the CTA's own start (min / median / max)")
    for i, nm in enumerate(names):
        col = rel[:, i][t[:, i] > 0]
        if col.numel():
            print(f"{nm:>20}: {int(col.min()):8d} {int(col.median()):8d} {int(col.max()):8d}")
    sys.exit(0)

print(f"# prefill attention: {B} x {QL} query tokens over {S} keys, {a.heads} q / {a.kv_heads} kv heads, "
      f"{flops / 1e12:.3f} TFLOP (causal)")
print("| kernel | ms | TFLOP/s | of measured bf16 peak |")
print("|---|---|---|---|")
res = {}
for name, flag in (("tcgen05 (prefill_umma)", True), ("mma.sync (paged_attention)", False)):
    attention_cuda.UMMA_PREFILL[0] = flag
    ms = timeit(lambda: attention_cuda.paged_attention_cuda(out, q, cache, bt, sl, qsl, D ** -0.5, QL, S))
    res[name] = out.float().clone()
    tf = flops / (ms * 1e-3) / 1e12
    print(f"| {name} | {ms:.3f} | {tf:.0f} | {tf / a.bf16_tflops:.2f} |", flush=True)
x, y = res.values()
print(f"max |difference| between the kernels: {(x - y).abs().max().item():.4g}")
check_status()
