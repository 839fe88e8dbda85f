"""Child process of ``test_failure_detection_cpu.py``: gloo ranks that all-reduce once per step under a RankMonitor.

Modes for the designated ``victim`` rank: ``leave`` - announces its exit after step 2 and exits between steps;
``vanish`` - exits after step 2 without a word.  Every other rank must learn of it on the host before its next
collective and report what it saw."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from vllm_kunlun_b200.parallel.health import RankLeft, RankMonitor, RankTimeout  # noqa: E402


def main():
    mode, victim, out = sys.argv[1], int(sys.argv[2]), sys.argv[3]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mon = RankMonitor.from_default_group(timeout=3.0)
    res = {"rank": rank, "steps": 0, "event": None}
    try:
        for step in range(1, 7):
            # host-side handshake BEFORE anything that waits on a peer: announce the step, then see every peer
            # announce it too (or learn that one left / stopped beating)
            mon.beat()
            mon.check(wait_for_step=step)
            t = torch.ones(4) * rank
            dist.all_reduce(t)
            assert t[0].item() == sum(range(world))
            res["steps"] = step
            if rank == victim and step == 2:
                if mode == "leave":
                    mon.leave("test: orderly exit")
                res["event"] = "exited"
                break
    except RankLeft as e:
        res["event"] = "RankLeft"
        res["message"] = str(e)
    except RankTimeout as e:
        res["event"] = "RankTimeout"
        res["message"] = str(e)
    with open(f"{out}.rank{rank}.json", "w") as fh:
        json.dump(res, fh)
    os._exit(0)  # no destroy_process_group: the peers are not all here any more


if __name__ == "__main__":
    main()
