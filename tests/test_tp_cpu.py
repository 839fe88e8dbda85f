"""Tensor / pipeline parallel plumbing on CPU ranks (gloo): TP=2 and PP=2 reproduce the single-rank tokens."""
import dataclasses
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from vllm_kunlun_b200.config import qwen2_0_5b


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg():
    return dataclasses.replace(qwen2_0_5b(), num_layers=2, vocab_size=512, hidden_size=128, num_heads=4, num_kv_heads=2,
                               head_dim=32, v_head_dim=32, rotary_dim=32, intermediate_size=256, max_position=1024)


def _prompts():
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 40, 7)]


def _full_state(cfg):
    """Deterministic full (unsharded) checkpoint in HF naming."""
    g = torch.Generator().manual_seed(7)
    sd = {}
    H, I = cfg.hidden_size, cfg.intermediate_size
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    sd["model.embed_tokens.weight"] = r(cfg.vocab_size, H)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = 1 + r(H)
        sd[p + "post_attention_layernorm.weight"] = 1 + r(H)
        sd[p + "self_attn.q_proj.weight"] = r(cfg.q_size, H)
        sd[p + "self_attn.k_proj.weight"] = r(cfg.kv_size, H)
        sd[p + "self_attn.v_proj.weight"] = r(cfg.kv_size, H)
        sd[p + "self_attn.q_proj.bias"] = r(cfg.q_size)
        sd[p + "self_attn.k_proj.bias"] = r(cfg.kv_size)
        sd[p + "self_attn.v_proj.bias"] = r(cfg.kv_size)
        sd[p + "self_attn.o_proj.weight"] = r(H, cfg.q_size)
        sd[p + "mlp.gate_proj.weight"] = r(I, H)
        sd[p + "mlp.up_proj.weight"] = r(I, H)
        sd[p + "mlp.down_proj.weight"] = r(H, I)
    sd["model.norm.weight"] = 1 + r(H)
    return sd


def _run(rank, world, port, tp, pp, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from vllm_kunlun_b200 import LLM, SamplingParams
    cfg = _cfg()
    llm = LLM(cfg, device="cpu", tensor_parallel_size=tp, pipeline_parallel_size=pp, block_size=16, max_model_len=128,
              max_num_seqs=4, num_gpu_blocks=64)
    with torch.inference_mode():
        llm.engine.runner.model.load_weights(_full_state(cfg).items())
    outs = llm.generate(_prompts(), SamplingParams(max_tokens=8, ignore_eos=True))
    if rank == world - 1:
        q.put([o.token_ids for o in outs])
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


def _launch(tp, pp):
    world = tp * pp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run, args=(r, world, port, tp, pp, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _q
    import time
    out, t0 = None, time.time()
    while out is None:
        try:
            out = q.get(timeout=2)
        except _q.Empty:
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            if dead or time.time() - t0 > 300:
                for p in procs:
                    p.kill()
                raise AssertionError(f"ranks failed or timed out: exit codes {[p.exitcode for p in procs]}")
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


@pytest.mark.parametrize("tp,pp", [(2, 1), (1, 2), (4, 1)])
def test_parallel_matches_single(tp, pp):
    ref = _launch(1, 1)
    assert _launch(tp, pp) == ref


def _serve_rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.entrypoints.openai_server import EngineLoop, build_app
    cfg = _cfg()
    llm = LLM(cfg, device="cpu", tensor_parallel_size=world, block_size=16, max_model_len=128, max_num_seqs=4,
              num_gpu_blocks=64)
    with torch.inference_mode():
        llm.engine.runner.model.load_weights(_full_state(cfg).items())
    if rank > 0:
        EngineLoop(llm).run_follower()  # returns when rank 0 stops
    else:
        from fastapi.testclient import TestClient
        app = build_app(llm, "tiny")
        with TestClient(app) as c:
            texts = [c.post("/v1/completions", json={"prompt": p, "max_tokens": 8, "temperature": 0.0,
                                                     "ignore_eos": True}).json()["choices"][0]["text"]
                     for p in _prompts()]
        app.state.engine_loop.stop()
        q.put([[int(t) for t in s.split()] for s in texts])
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


def test_http_server_over_two_tp_ranks():
    """Rank 0 serves HTTP and broadcasts each batch of new requests; rank 1 mirrors the steps.  The tokens equal
    the single-process engine's."""
    want = _launch(1, 1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_serve_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        got = q.get(timeout=180)
    except Exception:
        for p in procs:
            p.kill()
        raise
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want


def _run_dp(rank, world, port, tp, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from vllm_kunlun_b200 import LLM, SamplingParams
    cfg = _cfg()
    dp = world // tp
    llm = LLM(cfg, device="cpu", tensor_parallel_size=tp, data_parallel_size=dp, block_size=16, max_model_len=128,
              max_num_seqs=4, num_gpu_blocks=64)
    with torch.inference_mode():
        llm.engine.runner.model.load_weights(_full_state(cfg).items())
    st = llm.engine.pstate
    assert st.dp_size == dp and st.tp_size == tp and st.dp_rank == rank // tp
    # every replica serves its own share of the prompts; replica 1 gets one prompt fewer (different step counts)
    mine = _prompts()[st.dp_rank::dp]
    outs = llm.generate(mine, SamplingParams(max_tokens=8, ignore_eos=True))
    if st.tp_rank == tp - 1:
        q.put((st.dp_rank, [o.token_ids for o in outs]))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


@pytest.mark.parametrize("tp,dp", [(1, 2), (2, 2)])
def test_data_parallel_replicas_serve_their_own_requests(tp, dp):
    """``data_parallel_size`` replicas of ``tensor_parallel_size`` ranks schedule independently (different numbers of
    requests and steps) and give the single-rank tokens."""
    ref = _launch(1, 1)
    world = tp * dp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run_dp, args=(r, world, port, tp, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(dp))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for d in range(dp):
        assert got[d] == ref[d::dp], d
