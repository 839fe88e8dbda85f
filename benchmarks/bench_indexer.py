"""Lightning-indexer scoring of a prefill chunk: the tcgen05 kernel (csrc/attention/indexer_umma.cu) against the
mma.sync kernel (csrc/attention/indexer.cu), plus the top-2048 selection.  CUDA events, 2 warm-ups, median of 5.

    python benchmarks/bench_indexer.py                       # one 8192-token chunk at 32768 keys
    python benchmarks/bench_indexer.py --q-len 2048 --ctx 0
"""
import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200.ops import _ext  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status  # noqa: E402
from vllm_kunlun_b200.ops.mla_cuda import indexer_row_len  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--q-len", type=int, default=8192)
ap.add_argument("--ctx", type=int, default=24576)
ap.add_argument("--topk", type=int, default=2048)
a = ap.parse_args()
dev, bs, H = "cuda", 64, 64
T, S = a.q_len, a.ctx + a.q_len
nb = -(-S // bs)
cache = torch.randint(0, 255, (nb + 1, bs, 132), dtype=torch.uint8, device=dev)
cache.view(nb + 1, bs * 132)[:, bs * 128:].view(torch.float32).fill_(0.01)     # finite key scales
cache.view(nb + 1, bs * 132)[:, : bs * 128].clamp_(max=0x7e)                    # no e4m3 NaN codes (0x7f / 0xff)
bt = (torch.arange(nb, device=dev, dtype=torch.int32) + 1).view(1, nb)
sl = torch.tensor([S], device=dev, dtype=torch.int32)
qsl = torch.tensor([0, T], device=dev, dtype=torch.int32)
req = torch.zeros(T, device=dev, dtype=torch.int32)
q = torch.randint(0, 0x7e, (T, H, 128), dtype=torch.uint8, device=dev)
w = (torch.rand(T, H, device=dev) * 0.01).contiguous()
ld = -(-S // 512) * 512
logits = torch.empty(T, ld, device=dev)
row_len = indexer_row_len(sl, qsl, req, T)
out = torch.empty(T, a.topk, dtype=torch.int32, device=dev)
C = _ext.C()
flops = 2.0 * H * 128 * sum(a.ctx + r + 1 for r in range(T))


def timeit(fn, it=5):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(it):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


print(f"# indexer: {T} query tokens x 64 heads over {S} keys, {flops / 1e12:.2f} TFLOP (causal, fp8)")
print("| kernel | ms | TFLOP/s |")
print("|---|---|---|")
ms = timeit(lambda: C.indexer_logits_umma(logits, q, w, cache, bt, sl, qsl, T, 0))
a_ = logits[:, :S].clone()
print(f"| indexer_logits_umma_kernel (tcgen05, kind::f8f6f4) | {ms:.3f} | {flops / ms / 1e9:.0f} |", flush=True)
ms = timeit(lambda: C.indexer_logits(logits, q, w, cache, bt, sl, qsl, req, 0))
b_ = logits[:, :S].clone()
print(f"| indexer_logits_kernel (mma.sync e4m3) | {ms:.3f} | {flops / ms / 1e9:.0f} |", flush=True)
ms = timeit(lambda: C.topk_rows(out, logits, row_len))
print(f"| topk_rows_kernel (top-{a.topk}, row resident in shared memory) | {ms:.3f} | - |", flush=True)
mask = torch.arange(S, device=dev).unsqueeze(0) < row_len.unsqueeze(1)
d = torch.where(mask, (a_ - b_).abs(), torch.zeros_like(a_)).max().item()
print(f"max |difference| on visible keys: {d:.4g} (values up to {b_[mask].abs().max().item():.4g})")
check_status()
