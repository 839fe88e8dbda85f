"""Expert-parallel token exchange: the library baseline on gloo ranks reproduces the single-process MoE."""
import os
import socket

import torch
import torch.multiprocessing as mp

from vllm_kunlun_b200 import ops


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _problem(world, T=9, H=128, I=64, E=8, k=3):
    g = torch.Generator().manual_seed(0)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.1
    w2 = torch.randn(E, H, I, generator=g) * 0.1
    xs = [torch.randn(T, H, generator=g) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g) for _ in range(world)]
    return w13, w2, xs, logits, k


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    import torch.distributed as dist
    from vllm_kunlun_b200.parallel.ep_a2a import EPLibraryBaseline
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w13, w2, xs, logits, k = _problem(world)
    E = w13.shape[0]
    el = E // world
    wts, ids = ops.moe_route(logits[rank], k, "softmax", True)
    ep = EPLibraryBaseline(dist.group.WORLD, rank, world, E)
    out = ep.moe(xs[rank], ids, wts, w13[rank * el:(rank + 1) * el], w2[rank * el:(rank + 1) * el])
    q.put((rank, out.tolist()))
    dist.barrier()


def test_library_baseline_matches_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    w13, w2, xs, logits, k = _problem(world)
    for r in range(world):
        wts, ids = ops.moe_route(logits[r], k, "softmax", True)
        want = ops.fused_moe(xs[r], w13, w2, wts, ids)
        torch.testing.assert_close(torch.tensor(got[r]), want, atol=1e-5, rtol=1e-5)
