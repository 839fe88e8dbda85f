"""Decode context parallelism (MLA latent cache interleaved over ranks) on gloo ranks."""
import os
import socket

import torch
import torch.multiprocessing as mp

from vllm_kunlun_b200.attention.dcp import dcp_slot, local_context_len


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_interleaved_layout_arithmetic():
    pos = torch.arange(0, 11)
    for dcp in (2, 4):
        total = sum(local_context_len(pos, dcp, r) for r in range(dcp))
        assert total.tolist() == (pos + 1).tolist()  # every visible token is on exactly one rank
        for r in range(dcp):  # closed form: an equal share plus one for the ranks holding the remainder
            L = pos + 1
            assert local_context_len(pos, dcp, r).tolist() == (L // dcp + (r < L % dcp).long()).tolist()
    blocks = [7, 3]
    got = [dcp_slot(p, blocks, 4, 2, 1) for p in range(12)]
    assert got == [-1, 28, -1, 29, -1, 30, -1, 31, -1, 12, -1, 13]


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from test_deepseek_cpu import _cfg, _prompts
    from vllm_kunlun_b200 import LLM, SamplingParams
    outs = {}
    for dcp in (1, 2):
        llm = LLM(_cfg(), device="cpu", tensor_parallel_size=2, decode_context_parallel_size=dcp, block_size=64,
                  max_model_len=256, max_num_seqs=4, num_gpu_blocks=16, max_num_batched_tokens=48)
        outs[dcp] = [o.token_ids for o in llm.generate(_prompts(), SamplingParams(max_tokens=8, ignore_eos=True))]
    if rank == 0:
        q.put(outs)
    torch.distributed.barrier()


def test_dcp2_matches_plain_tp2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert outs[1] == outs[2], outs
