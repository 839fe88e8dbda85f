"""Process-group bookkeeping: one process per GPU, ``torch.distributed`` for the plumbing.

The reference relies on upstream vLLM's ``GroupCoordinator`` objects (world / TP / PP / EP / DP /
DCP) and only swaps the communicator class (``vllm_kunlun/platforms/kunlun.py:335-340``,
``vllm_kunlun/distributed/kunlun_communicator.py:12-86``).  Here the groups are created directly.
Rank layout is ``[dp][pp][tp]`` with TP innermost so a TP group sits on NVLink-adjacent ranks;
the EP group spans ``dp x tp`` ranks of one pipeline stage.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    tp_size: int = 1
    tp_rank: int = 0
    pp_size: int = 1
    pp_rank: int = 0
    dp_size: int = 1
    dp_rank: int = 0
    ep_size: int = 1
    ep_rank: int = 0
    dcp_size: int = 1
    dcp_rank: int = 0
    tp_group: Optional[object] = None
    pp_group: Optional[object] = None
    dp_group: Optional[object] = None
    ep_group: Optional[object] = None
    dcp_group: Optional[object] = None
    cpu_group: Optional[object] = None  # gloo group for host-side control (heartbeats, handle exchange)
    tp_comm: Optional[object] = None  # DeviceCommunicator
    ep_comm: Optional[object] = None
    pp_comm: Optional[object] = None
    dcp_comm: Optional[object] = None
    extras: dict = field(default_factory=dict)

    @property
    def is_first_pp(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp(self) -> bool:
        return self.pp_rank == self.pp_size - 1


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def set_state(st: ParallelState) -> None:
    global _STATE
    _STATE = st


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> tuple[int, int, int]:
    """Join the default process group from ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*``."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


def _new_groups(rank_lists, backend=None):
    mine = None
    for ranks in rank_lists:
        g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
        if dist.get_rank() in ranks:
            mine = (g, ranks)
    return mine


def initialize_model_parallel(tp: int = 1, pp: int = 1, dp: int = 1, ep: bool = False, dcp: int = 1,
                              device: str = "cpu", with_cpu_group: bool = True,
                              fused_collectives: bool = True) -> ParallelState:
    """Create TP / PP / DP / EP / DCP groups and their communicators."""
    from .. import envs
    fused_collectives = fused_collectives and envs.B200_PEER_COLLECTIVES
    from .communicator import DeviceCommunicator

    if not dist.is_initialized():
        st = ParallelState()
        set_state(st)
        return st
    world, rank = dist.get_world_size(), dist.get_rank()
    assert world == tp * pp * dp, f"world {world} != tp {tp} * pp {pp} * dp {dp}"
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    st = ParallelState(world_size=world, rank=rank, local_rank=local, tp_size=tp, pp_size=pp, dp_size=dp,
                       dcp_size=dcp)
    st.tp_rank = rank % tp
    st.pp_rank = (rank // tp) % pp
    st.dp_rank = rank // (tp * pp)
    grid = torch.arange(world).reshape(dp, pp, tp)
    tp_lists = [grid[d, p, :].tolist() for d in range(dp) for p in range(pp)]
    pp_lists = [grid[d, :, t].tolist() for d in range(dp) for t in range(tp)]
    dp_lists = [grid[:, p, t].tolist() for p in range(pp) for t in range(tp)]
    ep_lists = [grid[:, p, :].reshape(-1).tolist() for p in range(pp)]
    g = _new_groups(tp_lists)
    st.tp_group, tp_ranks = g
    st.pp_group, pp_ranks = _new_groups(pp_lists)
    st.dp_group, dp_ranks = _new_groups(dp_lists)
    if ep:
        st.ep_group, ep_ranks = _new_groups(ep_lists)
        st.ep_size = len(ep_ranks)
        st.ep_rank = ep_ranks.index(rank)
    if dcp > 1:
        assert tp % dcp == 0
        dcp_lists = [r[i:i + dcp] for r in tp_lists for i in range(0, tp, dcp)]
        st.dcp_group, dcp_ranks = _new_groups(dcp_lists)
        st.dcp_rank = dcp_ranks.index(rank)
    if with_cpu_group and world > 1:
        st.cpu_group = dist.new_group(list(range(world)), backend="gloo")
    if tp > 1:
        st.tp_comm = DeviceCommunicator(st.tp_group, tp_ranks, device, name="tp",
                                        enable_peer=fused_collectives, cpu_group=st.cpu_group)
    if ep and st.ep_size > 1:
        st.ep_comm = (st.tp_comm if st.ep_size == tp and dp == 1 else
                      DeviceCommunicator(st.ep_group, ep_ranks, device, name="ep",
                                         enable_peer=fused_collectives, cpu_group=st.cpu_group))
    if pp > 1:
        st.pp_comm = DeviceCommunicator(st.pp_group, pp_ranks, device, name="pp", enable_peer=False)
    if dcp > 1:
        st.dcp_comm = DeviceCommunicator(st.dcp_group, dcp_ranks, device, name="dcp", enable_peer=False)
    set_state(st)
    return st


def destroy_model_parallel() -> None:
    st = get_state()
    for c in (st.tp_comm, st.ep_comm, st.pp_comm, st.dcp_comm):
        if c is not None:
            c.destroy()
    set_state(ParallelState())
