"""Worker entry points for the multi-GPU tests (launched with ``python -m torch.distributed.run``).
Each worker writes ``<out>.rank<r>.json`` and leaves through ``os._exit`` after an orderly teardown."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def allreduce(rank, world):
    from vllm_kunlun_b200.ops.reference import basic as rb
    from vllm_kunlun_b200.parallel import state as ps
    ps.init_distributed("nccl")
    st = ps.initialize_model_parallel(tp=world, device=f"cuda:{rank}")
    peer = st.tp_comm.peer
    assert peer is not None
    dev = f"cuda:{rank}"
    worst = 0.0
    cases = [(16, 4096, torch.bfloat16), (1, 4096, torch.bfloat16), (33, 7168, torch.bfloat16),
             (200, 2048, torch.float16), (5, 1024, torch.float32)] * 3
    for it, (rows, H, dt) in enumerate(cases):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(rows, H, device=dev, generator=g).to(dt)
        ref = x.clone().float()
        dist.all_reduce(ref)
        out = peer.all_reduce(x)
        worst = max(worst, (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6))
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree bitwise"
        if dt != torch.float32:
            res = torch.randn(rows, H, device=dev, generator=torch.Generator(device=dev).manual_seed(it)).to(dt)
            w = torch.randn(H, device=dev, generator=torch.Generator(device=dev).manual_seed(it + 1)).to(dt)
            xo, ro = peer.all_reduce_add_rmsnorm(x.clone(), res.clone(), w, 1e-5)
            eo, er = rb.add_rmsnorm(ref.to(dt).cpu(), res.cpu(), w.cpu(), 1e-5)
            assert (ro.float().cpu() - er.float()).abs().max() < 0.05 * (er.float().abs().max() + 1)
            assert (xo.float().cpu() - eo.float()).abs().max() < 0.05 * (eo.float().abs().max() + 1)
    torch.cuda.synchronize()
    peer.check_status()
    return {"worst_rel_err": worst}


def engine(rank, world, fused):
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import llama_3_1_8b, tiny
    cfg = tiny(llama_3_1_8b(), num_layers=2, vocab_size=2048, hidden_size=1024, num_heads=8, num_kv_heads=2,
               head_dim=128, intermediate_size=2048, max_position=4096)
    llm = LLM(cfg, device="cuda", tensor_parallel_size=world, block_size=64, max_model_len=512, max_num_seqs=4,
              num_gpu_blocks=64, fused_collectives=bool(int(fused)), seed=5)
    # 192 + 64 = 256 prompt tokens in the first step: a multiple of world * 64, so the fused
    # GEMM+reduce-scatter / all-gather+GEMM path serves the prefill
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (192, 64)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    torch.cuda.synchronize()
    peer = llm.engine.pstate.tp_comm.peer
    launches = 0
    if int(fused):
        assert peer is not None and peer.launches > 0
        peer.check_status()
        launches = peer.launches
        assert getattr(peer, "sp_calls", 0) > 0, "fused GEMM+collective path was not taken"
    return {"tokens": [o.token_ids for o in outs], "peer_launches": launches}


if __name__ == "__main__":
    name, out = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    code = 0
    try:
        res = {"allreduce": allreduce, "engine": engine}[name](rank, world, *sys.argv[3:])
    except Exception:  # noqa: BLE001
        import traceback
        res = {"error": traceback.format_exc()}
        code = 1
    with open(f"{out}.rank{rank}.json", "w") as f:
        json.dump(res, f)
    # Orderly exit: every rank reaches the barrier, then leaves without tearing NCCL down (captured
    # CUDA graphs may still reference the communicator; process exit releases everything).
    try:
        if code == 0:
            torch.cuda.synchronize()
            dist.barrier(device_ids=[torch.cuda.current_device()])
    finally:
        sys.stdout.flush()
        os._exit(code)
