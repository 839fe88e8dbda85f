"""Failure detection without a GPU fault: failures are made on the host (a rank that leaves between steps, a rank
that vanishes) and the survivors must find out before their next collective instead of hanging in it."""
import json
import os
import socket
import subprocess
import sys
import tempfile

import pytest

from vllm_kunlun_b200.parallel.health import RankLeft, RankMonitor, RankTimeout

HERE = os.path.dirname(os.path.abspath(__file__))


class FakeStore:
    """The three c10d store calls the monitor uses, on a dict."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_monitor_sees_orderly_leave_and_missing_heartbeat():
    store = FakeStore()
    a, b, c = (RankMonitor(store, r, 3, timeout=0.05) for r in range(3))
    for m in (a, b, c):
        m.beat()
    a.check(wait_for_step=1)                       # everybody reached step 1
    b.beat(); c.beat()
    with pytest.raises(RankTimeout, match=r"\[0\]"):
        b.check(wait_for_step=2)                   # rank 0 never announced step 2
    c.leave("maintenance")
    with pytest.raises(RankLeft, match="maintenance"):
        a.check()
    with pytest.raises(RankLeft):
        b.check(wait_for_step=2)                   # a leave wins over waiting for the heartbeat
    assert a.peers_left() == {2: "maintenance"} and c.peers_left() == {}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("mode,expect", [("leave", "RankLeft"), ("vanish", "RankTimeout")])
def test_gloo_ranks_learn_on_the_host_that_a_peer_is_gone(mode, expect):
    world, victim = 3, 2
    out = os.path.join(tempfile.mkdtemp(), "res")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "health_worker.py"),
           mode, str(victim), out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
    res = []
    for k in range(world):
        path = f"{out}.rank{k}.json"
        assert os.path.exists(path), f"rank {k} wrote no result\n{r.stdout[-2000:]}\n{r.stderr[-3000:]}"
        res.append(json.load(open(path)))
    assert res[victim]["event"] == "exited" and res[victim]["steps"] == 2
    for k in range(world):
        if k != victim:
            # the survivors finished step 2 with the victim, then stopped BEFORE the third all-reduce
            assert res[k]["event"] == expect, res[k]
            assert res[k]["steps"] == 2, res[k]
            assert str(victim) in res[k]["message"]
