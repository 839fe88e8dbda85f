"""Tensor-parallel MLP block, fused peer-memory path vs the NCCL + separate-kernel path.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/bench_fused_tp.py [--tokens 8192] [--hidden 4096] [--inter 14336]

Chain timed per iteration (what one decoder layer's MLP half does under TP=N):
    down_proj partial GEMM -> reduce (+residual) -> RMSNorm -> gather -> gate_up GEMM
fused : GEMM with reduce-scatter epilogue -> rs_norm_ag kernel -> GEMM whose producer waits per tile
nccl  : GEMM -> NCCL all-reduce -> add+RMSNorm kernel -> GEMM
CUDA events on the launching stream, max over ranks.  The roofline is the slower of the FLOPs at the
measured GEMM peak and the bytes that must cross NVLink at 770 GB/s per direction."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200 import ops  # noqa: E402
from vllm_kunlun_b200.ops import gemm_cuda  # noqa: E402
from vllm_kunlun_b200.parallel import state as ps  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world, local = ps.init_distributed("nccl")
    torch.cuda.set_device(local)
    st = ps.initialize_model_parallel(tp=world, device=f"cuda:{local}")
    peer = st.tp_comm.peer
    T, H, I = a.tokens, a.hidden, a.inter // world
    peer.sp_init(T, H, torch.bfloat16)
    gemm_cuda.PEER = peer
    dev = f"cuda:{local}"
    g = torch.Generator(device=dev).manual_seed(rank)
    act = (torch.randn(T, I, device=dev, generator=g) * 0.5).bfloat16()
    w_down = (torch.randn(H, I, device=dev, generator=g) * 0.02).bfloat16()
    w_gu = (torch.randn(2 * I, H, device=dev, generator=g) * 0.02).bfloat16()
    res = torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).bfloat16()
    wn = torch.ones(H, device=dev, dtype=torch.bfloat16)
    out_f = torch.empty(T, 2 * I, device=dev, dtype=torch.bfloat16)
    out_n = torch.empty(T, 2 * I, device=dev, dtype=torch.bfloat16)

    def fused():
        h = peer.gemm_rs(act, w_down)
        x = peer.rs_norm_ag(h, res_f, wn, 1e-5)
        gemm_cuda.gemm_bf16(x, w_gu, out=out_f)

    def nccl():
        y = gemm_cuda.gemm_bf16(act, w_down)
        dist.all_reduce(y)
        x, _ = ops.add_rmsnorm(y, res_n, wn, 1e-5)
        gemm_cuda.gemm_bf16(x, w_gu, out=out_n)

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier(device_ids=[local])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    res_f, res_n = res.clone(), res.clone()
    fused(); nccl()
    torch.cuda.synchronize()
    # numerics: same block, two implementations (first call, identical residuals)
    err = (out_f.float() - out_n.float()).abs().max().item() / (out_n.float().abs().max().item() + 1e-6)
    res_f, res_n = res.clone(), res.clone()
    ms_f = timeit(fused)
    ms_n = timeit(nccl)
    peer.check_status()
    gemm_cuda.check_status()
    if rank == 0:
        peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json"))) \
            if os.path.exists(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0}
        flops = 2.0 * T * H * I + 2.0 * T * (2 * I) * H
        t_compute = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
        bytes_out = (world - 1) / world * T * H * 2  # reduce-scatter send = all-gather receive, per direction
        t_link = 2 * bytes_out / 770e9 * 1e3
        roof = max(t_compute, t_link)
        print(json.dumps({"bench": "tp_mlp_block", "world": world, "tokens": T, "hidden": H, "inter_per_rank": I,
                          "fused_ms": round(ms_f, 4), "nccl_ms": round(ms_n, 4), "speedup": round(ms_n / ms_f, 3),
                          "rel_err_vs_nccl": round(err, 5), "roofline_ms": round(roof, 4),
                          "compute_ms_at_peak": round(t_compute, 4), "nvlink_ms_at_770GBs": round(t_link, 4),
                          "fused_frac_of_roofline": round(roof / ms_f, 3)}), flush=True)
    torch.cuda.synchronize()
    dist.barrier(device_ids=[local])
    os._exit(0)


if __name__ == "__main__":
    main()
