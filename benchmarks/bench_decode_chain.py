"""In-graph cost of every kernel of a dense decode layer.

A decode step is a chain of small dependent kernels; timing one kernel alone (launch to completion,
cold) hides what matters in a step, which is how long the chain advances per kernel when the
launches are already queued (CUDA graph, programmatic dependent launch).  This script builds L
layers' worth of distinct weights (so every layer streams its weights from HBM, as a model does),
captures chains of the per-rank kernels of a tensor-parallel dense decoder and replays them:

    python benchmarks/bench_decode_chain.py --tp 1            # per-rank shapes at TP=1
    python benchmarks/bench_decode_chain.py --tp 8 --chains full,gemm4,qkv,o,gate_up,down,norm,rope,attn

Each chain is timed with CUDA events around ``--iters`` graph replays after warm-up; the figure is
microseconds per layer (per kernel for single-kernel chains) next to the bytes the kernel must move
divided by the measured copy bandwidth.  Collectives are not part of the chain (one GPU).
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200 import ops  # noqa: E402
from vllm_kunlun_b200.ops.attention_cuda import AttnWorkspace  # noqa: E402
from vllm_kunlun_b200.ops.gemm_cuda import check_status, interleave_gate_up  # noqa: E402
from vllm_kunlun_b200.ops.reference.basic import build_cos_sin_cache  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--tp", type=int, default=1)
ap.add_argument("--layers", type=int, default=32)
ap.add_argument("--batch", type=int, default=16)
ap.add_argument("--ctx", type=int, default=3072)
ap.add_argument("--hidden", type=int, default=4096)
ap.add_argument("--heads", type=int, default=32)
ap.add_argument("--kv-heads", type=int, default=8)
ap.add_argument("--inter", type=int, default=14336)
ap.add_argument("--iters", type=int, default=20)
ap.add_argument("--chains", default="full,gemm4,qkv,o,gate_up,down,norm,rope,attn")
ap.add_argument("--hbm-gbs", type=float, default=6548.5)
ap.add_argument("--attn-splits", type=int, default=0, help="force the split-KV count of decode attention (0 = planner)")
ap.add_argument("--json", default=None)
a = ap.parse_args()

dev = torch.device("cuda")
dt = torch.bfloat16
tp, L, B, H, D = a.tp, a.layers, a.batch, a.hidden, 128
hq, hkv = a.heads // tp, max(1, a.kv_heads // tp)
inter = a.inter // tp
qkv_n = (hq + 2 * hkv) * D
g = torch.Generator(device=dev).manual_seed(0)


def rnd(*shape, std=0.02):
    return (torch.randn(*shape, device=dev, generator=g, dtype=torch.float32) * std).to(dt)


W = {"qkv": [rnd(qkv_n, H) for _ in range(L)], "o": [rnd(H, hq * D) for _ in range(L)],
     "gate_up": [interleave_gate_up(rnd(2 * inter, H)) for _ in range(L)], "down": [rnd(H, inter) for _ in range(L)]}
norm_w = torch.ones(H, device=dev, dtype=dt)
bs = 64
blocks_per_seq = (a.ctx + 1 + bs - 1) // bs
nblk = B * blocks_per_seq
kv = [rnd(nblk, 2, hkv, bs, D, std=1.0) for _ in range(L)]
block_tables = torch.arange(nblk, device=dev, dtype=torch.int32).reshape(B, blocks_per_seq)
seq_lens = torch.full((B,), a.ctx + 1, device=dev, dtype=torch.int32)
qsl = torch.arange(B + 1, device=dev, dtype=torch.int32)
positions = torch.full((B,), a.ctx, device=dev, dtype=torch.int64)
slot_mapping = (block_tables[:, -1].long() * bs + a.ctx % bs)
cos_sin = build_cos_sin_cache(D, a.ctx + 64, 5e5, None).to(dev)
ws = AttnWorkspace(B, hq, D, 16, dev)

x = rnd(B, H, std=1.0)
res = rnd(B, H, std=1.0)
qkv_buf = rnd(B, qkv_n, std=1.0)
q_buf = rnd(B, hq, D, std=1.0)
o_buf = rnd(B, hq * D, std=1.0)
act_buf = rnd(B, inter, std=1.0)
scale = D ** -0.5


def k_norm(l):
    ops.add_rmsnorm(x, res, norm_w, 1e-5)


def k_qkv(l):
    return ops.linear(x, W["qkv"][l], out=qkv_buf)


def k_rope(l):
    return ops.qkv_split_norm_rope_cache(qkv_buf, positions, cos_sin, None, None, 1e-5, hq, hkv, D, True, kv[l],
                                         slot_mapping)


def k_attn(l):
    from vllm_kunlun_b200.ops.attention_cuda import paged_attention_cuda
    return paged_attention_cuda(o_buf.view(B, hq, D), q_buf, kv[l], block_tables, seq_lens, qsl, scale, 1, a.ctx + 64,
                                None, None, ws, a.attn_splits or None, stable_metadata=True)


def k_o(l):
    return ops.linear(o_buf, W["o"][l], out=x)


def k_gate_up(l):
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_bf16
    return gemm_bf16(x, W["gate_up"][l], None, out=act_buf, act="silu")


def k_down(l):
    return ops.linear(act_buf, W["down"][l], out=x)


CHAINS = {
    "full": [k_norm, k_qkv, k_rope, k_attn, k_o, k_norm, k_gate_up, k_down],
    "gemm4": [k_qkv, k_o, k_gate_up, k_down],
    "noattn": [k_norm, k_qkv, k_rope, k_o, k_norm, k_gate_up, k_down],
    "rope_attn": [k_rope, k_attn],
    "qkv": [k_qkv], "o": [k_o], "gate_up": [k_gate_up], "down": [k_down],
    "norm": [k_norm], "rope": [k_rope], "attn": [k_attn],
}
BYTES = {
    "qkv": qkv_n * H * 2, "o": H * hq * D * 2, "gate_up": 2 * inter * H * 2, "down": H * inter * 2,
    "norm": 0, "rope": 0, "attn": B * (a.ctx + 1) * hkv * D * 2 * 2,
}
BYTES["gemm4"] = BYTES["qkv"] + BYTES["o"] + BYTES["gate_up"] + BYTES["down"]
BYTES["full"] = BYTES["gemm4"] + BYTES["attn"]
BYTES["noattn"] = BYTES["gemm4"]
BYTES["rope_attn"] = BYTES["attn"]


def time_chain(fns):
    def run():
        for l in range(L):
            for f in fns:
                f(l)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        run()
        run()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / L)
    return statistics.median(ts), min(ts)


out = {"tp": tp, "layers": L, "batch": B, "ctx": a.ctx, "shapes": {"qkv": [B, qkv_n, H], "o": [B, H, hq * D],
                                                                       "gate_up": [B, 2 * inter, H], "down": [B, H, inter]}}
print(f"# per-rank shapes at TP={tp}: qkv {B}x{qkv_n}x{H}, o {B}x{H}x{hq * D}, gate_up {B}x{2 * inter}x{H}, "
      f"down {B}x{H}x{inter}; attention {B} x ctx {a.ctx} x {hkv} kv heads; {L} layers per graph")
print("| chain | us per layer (median) | min | bytes / measured HBM (us) |")
print("|---|---|---|---|")
with torch.inference_mode():
    for name in a.chains.split(","):
        med, mn = time_chain(CHAINS[name])
        ideal = BYTES[name] / (a.hbm_gbs * 1e3)
        out[name] = {"us": round(med, 2), "min_us": round(mn, 2), "ideal_us": round(ideal, 2)}
        print(f"| {name} | {med:.2f} | {mn:.2f} | {ideal:.2f} |", flush=True)
check_status()
if a.json:
    with open(a.json, "w") as fh:
        json.dump(out, fh)
