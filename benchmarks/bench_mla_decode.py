"""Dense paged MLA decode: the tcgen05 kernel (csrc/attention/mla_decode_umma.cu) against the mma.sync kernel
(csrc/attention/mla_attention.cu), timed in a CUDA-graph chain over ``--layers`` distinct latent caches (cold cache
rows, queued launches - as inside a decode step).

    python benchmarks/bench_mla_decode.py                      # 16 requests x 4096 context, 16 heads (TP=8 shard)
    python benchmarks/bench_mla_decode.py --heads 128 --qlen 2

Prints microseconds per launch and the fraction of the measured copy bandwidth that the latent-cache bytes
(``requests x context x 1152 B``, read once) correspond to.
"""
import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200.ops import mla_cuda  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--batch", type=int, default=16)
ap.add_argument("--ctx", type=int, default=4096)
ap.add_argument("--heads", type=int, default=16)
ap.add_argument("--qlen", type=int, default=1)
ap.add_argument("--layers", type=int, default=8)
ap.add_argument("--iters", type=int, default=20)
ap.add_argument("--hbm-gbs", type=float, default=6548.5)
ap.add_argument("--impl", default="umma,mma_sync")
ap.add_argument("--splits", type=int, default=0, help="0 = planned; negative = that many through the workspace")
ap.add_argument("--trace", action="store_true", help="print the tcgen05 kernel's phase timestamps (one launch)")
a = ap.parse_args()
dev, dt = "cuda", torch.bfloat16
B, N, q = a.batch, a.heads, a.qlen
bs = 64
nblk_per = -(-(a.ctx + q) // bs)
nblk = B * nblk_per
caches = [(torch.randn(nblk, bs, 576, device=dev) * 0.3).to(dt) for _ in range(a.layers)]
bt = torch.arange(nblk, device=dev, dtype=torch.int32).reshape(B, nblk_per)
sl = torch.full((B,), a.ctx + q, device=dev, dtype=torch.int32)
qsl = torch.arange(0, (B + 1) * q, q, device=dev, dtype=torch.int32)
qq = (torch.randn(B * q, N, 576, device=dev) * 0.3).to(dt)
bytes_ = B * (a.ctx + q) * 1152
if a.splits:
    _plan = mla_cuda.plan_mla_splits
    mla_cuda.plan_mla_splits = lambda *args, **kw: (abs(a.splits), a.splits > 0 and a.splits in (2, 4, 8))
R_ = 16 if N * q <= 16 else 32
print("# plan (splits, cluster merge):", mla_cuda.plan_mla_splits(B * -(-N // (R_ // q)), -(-(a.ctx + q) // 64), R_, dt, dev),
      "| resident clusters of 2/4/8:", [mla_cuda._max_clusters(R_, S, dt, dev) for S in (2, 4, 8)])


def run(impl):
    mla_cuda.UMMA_DECODE[0] = impl == "umma"

    def chain():
        for c in caches:
            mla_cuda.mla_attention_cuda(qq, c, bt, sl, qsl, 0.1, 512, q, a.ctx + q, stable_metadata=True)
    chain()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        chain()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / a.layers)
    return statistics.median(ts)


if a.trace:
    from vllm_kunlun_b200.ops import _ext
    C = _ext.C()
    tr = torch.zeros(24 << 14, dtype=torch.int64, device=dev)
    mla_cuda.UMMA_DECODE[0] = True
    with torch.inference_mode():
        for c in caches[:2]:   # the second launch has a predecessor, as inside a step
            tr.zero_()
            C.set_kernel_trace(tr)
            mla_cuda.mla_attention_cuda(qq, c, bt, sl, qsl, 0.1, 512, q, a.ctx + q, stable_metadata=True)
            torch.cuda.synchronize()
            C.set_kernel_trace(None)
    t = tr.view(-1, 24).cpu()
    t = t[t[:, 0] > 0]
    t0 = int(t[:, 0].min())
    names = ["start", "Q staged", "first S^T", "last P", "last P.V", "A / row sums", "B / ticket", "end",
             "t4 stage free", "t4 landed", "t4 S^T", "t4 P", "t4 P seen", "merge weights", "merge landed", "merge done",
             "rows ready", "partial stored", "fenced", "merge pass0 done"]
    print(f"# phase trace over {t.shape[0]} CTAs: ns after the first CTA's start (min / median / max)")
    for i, nm in enumerate(names):
        col = t[:, i][t[:, i] > 0] - t0
        if col.numel():
            print(f"{nm:>14}: {int(col.min()):7d} {int(col.median()):7d} {int(col.max()):7d}")
    sys.exit(0)

print(f"# MLA decode: {B} requests x ctx {a.ctx}, {N} heads, q_len {q}; latent bytes {bytes_ / 1e6:.1f} MB "
      f"= {bytes_ / (a.hbm_gbs * 1e3):.2f} us at {a.hbm_gbs} GB/s")
print("| kernel | us per launch | fraction of measured HBM bandwidth |")
print("|---|---|---|")
with torch.inference_mode():
    outs = {}
    for impl in a.impl.split(","):
        t = run(impl)
        outs[impl] = mla_cuda.mla_attention_cuda(qq, caches[0], bt, sl, qsl, 0.1, 512, q, a.ctx + q).float()
        print(f"| {impl} | {t:.2f} | {bytes_ / (t * 1e-6) / (a.hbm_gbs * 1e9):.3f} |", flush=True)
    if len(outs) == 2:
        x, y = outs.values()
        print(f"max |difference| between the kernels: {(x - y).abs().max().item():.4g}")
check_status()
