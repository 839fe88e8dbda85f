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
    # Low-latency path with the row width and the row count changing from call to call and no other
    # synchronisation between the calls: one call-wide epoch keeps every CTA of every rank on the same parity.
    shapes = [(16, 4096), (3, 1024), (32, 2048), (1, 4096), (16, 512), (8, 7168), (16, 4096), (2, 128)]
    xs, refs = [], []
    for it in range(48):
        rows, H = shapes[it % len(shapes)]
        g = torch.Generator(device=dev).manual_seed(7000 + 10 * it + rank)
        x = torch.randn(rows, H, device=dev, generator=g).to(torch.bfloat16)
        ref = x.clone().float()
        dist.all_reduce(ref)
        xs.append(x); refs.append(ref)
    torch.cuda.synchronize()
    dist.barrier()
    outs = [peer.all_reduce(x) for x in xs]  # 48 back-to-back launches
    torch.cuda.synchronize()
    for out, ref in zip(outs, refs):
        assert (out.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 0.02, "mixed-shape low-latency all-reduce"
    # Row-parallel decode GEMM that pushes its partials from the epilogue, then collect + residual + norm.
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_decode_push
    for it, (rows, N, K) in enumerate([(16, 4096, 512), (16, 4096, 1792), (5, 1024, 2048), (32, 2048, 256)] * 2):
        g = torch.Generator(device=dev).manual_seed(9000 + 10 * it + rank)
        x = torch.randn(rows, K, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        res = torch.randn(rows, N, device=dev, generator=torch.Generator(device=dev).manual_seed(it)).to(torch.bfloat16)
        nw = torch.randn(N, device=dev, generator=torch.Generator(device=dev).manual_seed(it + 1)).to(torch.bfloat16)
        part = (x.float() @ w.float().T).to(torch.bfloat16)
        ref = part.float()
        dist.all_reduce(ref)
        assert peer.can_push(rows, N, x.dtype)
        y = gemm_decode_push(x, w, peer)
        assert (y.float() - part.float()).abs().max() <= 0.01 * part.float().abs().max() + 0.02, "local partial"
        r2 = res.clone()
        xo, ro = peer.all_reduce_add_rmsnorm(y, r2, nw, 1e-5, pushed=True)
        eo, er = rb.add_rmsnorm(ref.to(torch.bfloat16).cpu(), res.cpu(), nw.cpu(), 1e-5)
        assert (ro.float().cpu() - er.float()).abs().max() < 0.02 * (er.float().abs().max() + 1), "pushed residual"
        assert (xo.float().cpu() - eo.float()).abs().max() < 0.03 * (eo.float().abs().max() + 1), "pushed norm"
        gathered = [torch.empty_like(xo) for _ in range(world)]
        dist.all_gather(gathered, xo.contiguous())
        assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree bitwise after the pushed GEMM"
    torch.cuda.synchronize()
    peer.check_status()
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    check_status()
    return {"worst_rel_err": worst}


def engine(rank, world, fused):
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import llama_3_1_8b, tiny
    cfg = tiny(llama_3_1_8b(), num_layers=2, vocab_size=2048, hidden_size=1024, num_heads=8, num_kv_heads=2,
               head_dim=128, intermediate_size=2048, max_position=4096)
    llm = LLM(cfg, device="cuda", tensor_parallel_size=world, block_size=64, max_model_len=1024, max_num_seqs=4,
              num_gpu_blocks=64, fused_collectives=bool(int(fused)), seed=5)
    # the prompt tokens of the first step add up to a multiple of world * 64, so the fused
    # GEMM+reduce-scatter / all-gather+GEMM path serves the prefill
    total = max(256, world * 64)
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist()
               for n in (total - 64, 64)]
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


def ep_a2a(rank, world, fp8):
    """Dispatch / combine over peer memory against the library baseline and the dense oracle."""
    import time

    from vllm_kunlun_b200 import ops
    from vllm_kunlun_b200.models.moe import _quant_block_device
    from vllm_kunlun_b200.parallel import state as ps
    from vllm_kunlun_b200.parallel.ep_a2a import EPAll2All, EPLibraryBaseline
    fp8 = bool(int(fp8))
    ps.init_distributed("nccl")
    st = ps.initialize_model_parallel(tp=world, device=f"cuda:{rank}")
    dev = f"cuda:{rank}"
    H, I, E, k, cap = 2048, 768, 128, 8, 2048
    el = E // world
    g = torch.Generator(device=dev).manual_seed(1234)  # same weights on every rank, each keeps its slice
    w13 = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05)
    w2 = (torch.randn(E, H, I, device=dev, generator=g) * 0.05)
    s13 = s2 = None
    if fp8:
        q13, q2, s13l, s2l = [], [], [], []
        for e in range(rank * el, (rank + 1) * el):
            a, b = _quant_block_device(w13[e])
            c, d = _quant_block_device(w2[e])
            q13.append(a), s13l.append(b), q2.append(c), s2l.append(d)
        lw13, lw2, s13, s2 = torch.stack(q13), torch.stack(q2), torch.stack(s13l), torch.stack(s2l)
    else:
        lw13 = w13[rank * el:(rank + 1) * el].to(torch.bfloat16).contiguous()
        lw2 = w2[rank * el:(rank + 1) * el].to(torch.bfloat16).contiguous()
    ep = EPAll2All(st.tp_comm, cap, H, k, E, fp8_payload=fp8)
    base = EPLibraryBaseline(st.tp_comm.group, rank, world, E)
    worst = 0.0
    for it, T in enumerate([64, 1, 300, 2048, 16, 16]):
        gr = torch.Generator(device=dev).manual_seed(77 * it + rank)
        x = torch.randn(T, H, device=dev, generator=gr).to(torch.bfloat16)
        logits = torch.randn(T, E, device=dev, generator=gr)
        wts, ids = ops.moe_route(logits, k, "softmax", True)
        add = torch.randn(T, H, device=dev, generator=gr).to(torch.bfloat16) if it % 2 else None
        got = ep.moe(x, ids, wts, lw13, lw2, "silu", None, None, s13, s2, addend=add, bound=T if it % 3 else None)
        want = base.moe(x, ids, wts, lw13, lw2, "silu", None, None, s13, s2, addend=add)
        torch.cuda.synchronize()
        ep.check_status()
        err = (got.float() - want.float()).abs().max().item() / (want.float().abs().max().item() + 1e-6)
        worst = max(worst, err)
    # uneven token counts, including a rank with none
    T = 0 if rank == 0 else 40 + rank
    gr = torch.Generator(device=dev).manual_seed(999 + rank)
    x = torch.randn(T, H, device=dev, generator=gr).to(torch.bfloat16)
    wts, ids = ops.moe_route(torch.randn(T, E, device=dev, generator=gr), k, "softmax", True) if T else (
        torch.zeros(0, k, device=dev), torch.zeros(0, k, dtype=torch.int32, device=dev))
    got = ep.moe(x, ids, wts, lw13, lw2, "silu", None, None, s13, s2, bound=40 + world)
    torch.cuda.synchronize()
    ep.check_status()
    if T and not fp8:
        dense = ops.fused_moe(x, w13.to(torch.bfloat16), w2.to(torch.bfloat16), wts, ids)
        worst = max(worst, (got.float() - dense.float()).abs().max().item() / (dense.float().abs().max().item() + 1e-6))
    # timing, device clock, max over ranks
    res = {"worst_rel_err": worst}
    for T in (16, 1024):
        gr = torch.Generator(device=dev).manual_seed(5 + rank)
        x = torch.randn(T, H, device=dev, generator=gr).to(torch.bfloat16)
        wts, ids = ops.moe_route(torch.randn(T, E, device=dev, generator=gr), k, "softmax", True)
        for name, impl in (("a2a", ep), ("lib", base)):
            kw = {"bound": T} if name == "a2a" else {}
            for _ in range(5):
                impl.moe(x, ids, wts, lw13, lw2, "silu", None, None, s13, s2, **kw)
            torch.cuda.synchronize()
            dist.barrier(device_ids=[rank])
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                impl.moe(x, ids, wts, lw13, lw2, "silu", None, None, s13, s2, **kw)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 20], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[f"{name}_ms_T{T}"] = round(t.item(), 4)
    ep.check_status()
    return res


def dcp_engine(rank, world):
    """MLA engine with the latent cache interleaved over the ranks (decode context parallel) vs plain TP."""
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import RopeScaling, deepseek_v3, tiny
    cfg = tiny(deepseek_v3(fp8=False), num_layers=3, first_dense_layers=1, vocab_size=1024, hidden_size=512,
               num_heads=16, num_kv_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=1024,
               num_experts=16, num_experts_per_tok=16, moe_intermediate_size=256, n_group=1, topk_group=1,
               max_position=2048, rope_scaling=RopeScaling(type="yarn", factor=4.0, original_max_position=512,
                                                           mscale=1.0, mscale_all_dim=1.0), num_mtp_layers=0)
    prompts = [torch.randint(0, 1024, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (150, 33, 70)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    res = {}
    for name, dcp, eager in (("tp", 1, True), ("dcp_eager", world, True), ("dcp_graph", world, False)):
        llm = LLM(cfg, device="cuda", tensor_parallel_size=world, decode_context_parallel_size=dcp, block_size=64,
                  max_model_len=512, max_num_seqs=4, num_gpu_blocks=32, seed=3, enforce_eager=eager)
        res[name] = [o.token_ids for o in llm.generate(prompts, sp)]
        torch.cuda.synchronize()
    return res


def sparse_mla_engine(rank, world):
    """Lightning indexer under TP: every rank scores a slice of the prefill tokens against its complete key cache
    and the selections are all-gathered.  The selections must be the same on all ranks and must match the
    replicated scoring up to near-ties (the q projection of a 264-row slice and of the 527-row batch may differ in
    the last bf16 bit, since the GEMM picks its split by the token count)."""
    from vllm_kunlun_b200.attention.metadata import AttentionMetadata
    from vllm_kunlun_b200.config import deepseek_v3, tiny
    from vllm_kunlun_b200.models.deepseek import Indexer
    from vllm_kunlun_b200.models.layers import get_cos_sin_cache
    from vllm_kunlun_b200.parallel import state as ps
    ps.init_distributed("nccl")
    ps.initialize_model_parallel(tp=world, device=f"cuda:{rank}")
    cfg = tiny(deepseek_v3(fp8=False, sparse=True), num_layers=1, vocab_size=1024, hidden_size=512, q_lora_rank=256,
               max_position=2048, index_topk=64)
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(11)   # the same weights and inputs on every rank
    idx = Indexer(cfg, torch.bfloat16, dev)
    for p_ in idx.parameters():
        p_.data.normal_(0, 0.05)
    idx.k_norm_weight.data.fill_(1.0)
    lens = [300, 77, 150]
    T, bs = sum(lens), 64
    hidden = torch.randn(T, 512, device=dev).bfloat16()
    q_c = torch.randn(T, 256, device=dev).bfloat16()
    nblk = [-(-n // bs) for n in lens]
    bt = torch.zeros(len(lens), max(nblk), dtype=torch.int32, device=dev)
    o = 1
    for b_, n in enumerate(nblk):
        bt[b_, :n] = torch.arange(o, o + n, dtype=torch.int32, device=dev)
        o += n
    pos = torch.cat([torch.arange(n, device=dev) for n in lens]).long()
    req = torch.cat([torch.full((n,), r, dtype=torch.int32, device=dev) for r, n in enumerate(lens)])
    slots = (bt[req.long(), (pos // bs)].long() * bs + pos % bs).long()
    qsl = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    cos_sin = get_cos_sin_cache(64, 2048, 10000.0, None, dev)
    res = {}
    for name, min_tokens in (("replicated", 1 << 30), ("sliced", 1)):
        Indexer.SP_MIN_TOKENS = min_tokens
        cache = torch.zeros(o, bs, 132, dtype=torch.uint8, device=dev)
        md = AttentionMetadata(num_tokens=T, num_reqs=len(lens), positions=pos, slot_mapping=slots, block_tables=bt,
                               seq_lens=sl, query_start_loc=qsl, max_query_len=max(lens), max_seq_len=max(lens),
                               num_prefills=len(lens), req_id_per_token=req)
        with torch.inference_mode():
            out = idx(hidden, q_c, pos, cos_sin, cache, md)
        torch.cuda.synchronize()
        res[name] = out.sort(-1).values.cpu().tolist()
    Indexer.SP_MIN_TOKENS = 64
    res["rows_that_differ"] = [i for i, (a, b) in enumerate(zip(res["sliced"], res["replicated"])) if a != b]
    return res


def ep_block(rank, world):
    """One sparse-MoE block on replicated tokens: dispatch / combine path against the replicated-token path."""
    os.environ["B200_EP_A2A"] = "1"
    os.environ["B200_EP_A2A_MAX_TOKENS"] = "1024"
    from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
    from vllm_kunlun_b200.models.moe import SparseMoEBlock
    from vllm_kunlun_b200.parallel import state as ps
    ps.init_distributed("nccl")
    st = ps.initialize_model_parallel(tp=world, ep=True, device=f"cuda:{rank}")
    dev = f"cuda:{rank}"
    cfg = tiny(qwen3_30b_a3b(fp8=False), num_layers=1, vocab_size=2048, hidden_size=1024, num_heads=8, num_kv_heads=2,
               head_dim=128, intermediate_size=1024, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256)
    worst = 0.0
    with torch.inference_mode():
        blk = SparseMoEBlock(cfg, torch.bfloat16, dev)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        for p in blk.parameters():
            p.data.copy_((torch.randn(p.shape, device=dev, generator=g) * 0.05).to(p.dtype))
        dist.broadcast(blk.gate.weight.data, 0)
        for T in (253, 4, 3, 2, 700):
            x = torch.randn(T, 1024, device=dev, generator=torch.Generator(device=dev).manual_seed(T)).to(torch.bfloat16)
            a2a = blk._a2a(x)
            assert a2a is not None
            ya = blk._forward_a2a(x, a2a).float()
            os.environ["B200_EP_A2A"] = "0"
            yb = blk(x).float()
            os.environ["B200_EP_A2A"] = "1"
            dist.all_reduce(ya)
            dist.all_reduce(yb)
            torch.cuda.synchronize()
            a2a.check_status()
            worst = max(worst, (ya - yb).abs().max().item() / (yb.abs().max().item() + 1e-6))
    return {"worst_rel_err": worst}


def ep_engine(rank, world, a2a):
    """Expert-parallel MoE engine: replicated-token path vs the dispatch / combine path, eager and captured."""
    os.environ["B200_EP_A2A_MAX_TOKENS"] = "1024"
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
    cfg = tiny(qwen3_30b_a3b(fp8=False), num_layers=2, vocab_size=2048, hidden_size=1024, num_heads=8, num_kv_heads=2,
               head_dim=128, intermediate_size=1024, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256,
               max_position=2048)
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (150, 33, 70)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    res = {}
    for name, env, eager in (("a2a_eager", "1", True), ("rep_eager", "0", True), ("a2a_graph", "1", False)):
        os.environ["B200_EP_A2A"] = env
        llm = LLM(cfg, device="cuda", tensor_parallel_size=world, enable_expert_parallel=True, block_size=64,
                  max_model_len=512, max_num_seqs=4, num_gpu_blocks=64, seed=11, enforce_eager=eager)
        res[name] = [o.token_ids for o in llm.generate(prompts, sp)]
        torch.cuda.synchronize()
        a2a = getattr(llm.engine.pstate, "ep_a2a", None)
        if env == "1":
            assert a2a is not None, "dispatch / combine path was not taken"
            a2a.check_status()
    return res


if __name__ == "__main__":
    name, out = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    code = 0
    try:
        res = {"allreduce": allreduce, "engine": engine, "ep_a2a": ep_a2a, "ep_engine": ep_engine, "ep_block": ep_block, "dcp_engine": dcp_engine,
               "sparse_mla_engine": sparse_mla_engine}[name](rank, world, *sys.argv[3:])
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
