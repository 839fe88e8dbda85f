"""Peer-memory collectives and the tensor-parallel engine on >= 2 GPUs of one node.  Ranks run as
child processes under ``torch.distributed.run`` with a hard timeout; NVLS is switched off (the
kernels use plain peer loads/stores)."""
import json
import os
import socket
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, name, *args, timeout=300):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = os.path.join(tempfile.mkdtemp(), "res")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "mg_workers.py"),
           name, out, *map(str, args)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    res = []
    for k in range(world):
        path = f"{out}.rank{k}.json"
        assert os.path.exists(path), f"rank {k} wrote no result\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
        res.append(json.load(open(path)))
    errs = [x["error"] for x in res if "error" in x]
    assert not errs, errs[0]
    return res


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_and_pushed_gemm(world):
    """One-shot / low-latency all-reduce (fixed and changing shapes, no library sync between calls) and the decode
    GEMM that pushes its partial sums from the epilogue, against NCCL sums; bit-equality across ranks."""
    res = _run(world, "allreduce")
    assert all(x["worst_rel_err"] < 0.02 for x in res), res


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_engine_fused_vs_nccl(world):
    a = _run(world, "engine", 1)
    b = _run(world, "engine", 0)
    assert all(a[0]["tokens"] == a[k]["tokens"] for k in range(world)), "ranks disagree"
    assert a[0]["peer_launches"] > 0
    # the peer-memory path (fp32 sum in rank order) and NCCL may differ in the last bf16 bit; most
    # greedy tokens must still agree
    fa, fb = sum(a[0]["tokens"], []), sum(b[0]["tokens"], [])
    assert sum(x == y for x, y in zip(fa, fb)) >= 0.7 * len(fa), (fa, fb)


@pytest.mark.parametrize("fp8", [0, 1])
def test_ep_dispatch_combine_2gpu(fp8):
    res = _run(2, "ep_a2a", fp8)
    tol = 0.08 if fp8 else 0.03
    assert all(x["worst_rel_err"] < tol for x in res), res
    print("EP timings", res[0])


def test_ep_block_a2a_vs_replicated_2gpu():
    res = _run(2, "ep_block")
    assert all(x["worst_rel_err"] < 0.03 for x in res), res


def test_ep_engine_a2a_vs_replicated_2gpu():
    a = _run(2, "ep_engine", 1, timeout=600)
    assert a[0] == a[1], "ranks disagree"
    flat = {k: sum(v, []) for k, v in a[0].items()}
    n = len(flat["rep_eager"])
    # the two paths add the expert outputs in different orders (bf16): most greedy tokens agree
    assert sum(x == y for x, y in zip(flat["a2a_eager"], flat["rep_eager"])) >= 0.7 * n, flat
    assert sum(x == y for x, y in zip(flat["a2a_graph"], flat["a2a_eager"])) >= 0.9 * n, flat


def test_dcp_engine_2gpu():
    a = _run(2, "dcp_engine", timeout=600)
    assert a[0] == a[1], "ranks disagree"
    flat = {k: sum(v, []) for k, v in a[0].items()}
    n = len(flat["tp"])
    assert sum(x == y for x, y in zip(flat["dcp_eager"], flat["tp"])) >= 0.7 * n, flat
    assert sum(x == y for x, y in zip(flat["dcp_graph"], flat["dcp_eager"])) >= 0.9 * n, flat


def test_sparse_mla_indexer_sliced_over_tp_2gpu():
    res = _run(2, "sparse_mla_engine")
    assert res[0]["sliced"] == res[1]["sliced"], "ranks disagree"
    differ = res[0]["rows_that_differ"]
    # a row may differ only through a near-tie at the selection boundary (the q projection of a slice and of the
    # whole batch can differ in the last bf16 bit)
    assert len(differ) <= 0.01 * len(res[0]["sliced"]), f"{len(differ)} rows differ: {differ[:40]}"
