"""Device communicator for one process group.

The reference's ``KunlunCommunicator`` (``vllm_kunlun/distributed/kunlun_communicator.py:12-86``)
turns every fast path off and calls plain ``torch.distributed``; it warms the group up with a
1-float all-reduce (``:36-40``) and its ``destroy`` is a no-op (``:62-64``).  This communicator keeps
NCCL for bootstrap, large collectives and pipeline send/recv, and adds a peer-memory path over
NVLink/NVSwitch (``symm_mem.PeerBuffers``) used by the hand-written one-shot all-reduce,
GEMM->reduce-scatter, all-gather->GEMM and EP dispatch/combine kernels.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.distributed as dist


class DeviceCommunicator:
    def __init__(self, group, ranks, device: str = "cpu", name: str = "tp", enable_peer: bool = True,
                 cpu_group=None, peer_bytes: int = 64 << 20):
        self.group = group
        self.ranks = list(ranks)
        self.world_size = len(self.ranks)
        self.rank_in_group = self.ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.name = name
        self.cpu_group = cpu_group
        self.peer = None
        self.disabled = False
        self._side_stream = None
        if self.world_size > 1:
            # Handshake: the first collective also forces NCCL to build its rings / NVLS trees.
            t = torch.zeros(1, device=self.device)
            dist.all_reduce(t, group=self.group)
            if self.device.type == "cuda":
                torch.cuda.synchronize()
                self._side_stream = torch.cuda.Stream()
                if enable_peer:
                    from .symm_mem import PeerBuffers
                    self.peer = PeerBuffers.create(self, peer_bytes)

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.peer is not None and not self.disabled and self.peer.can_one_shot(x):
            return self.peer.all_reduce(x)
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if dim < 0:
            dim += x.dim()
        x = x.contiguous()
        flat = torch.empty((self.world_size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x, group=self.group)
        if dim == 0:
            return flat
        out = flat.reshape((self.world_size,) + tuple(x.shape)).movedim(0, dim)
        shp = list(x.shape)
        shp[dim] *= self.world_size
        return out.reshape(shp)

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return x
        xm = x.movedim(dim, 0).contiguous()
        assert xm.shape[0] % self.world_size == 0
        out = torch.empty((xm.shape[0] // self.world_size,) + tuple(xm.shape[1:]), dtype=x.dtype,
                          device=x.device)
        if xm.is_cuda:
            dist.reduce_scatter_tensor(out, xm, group=self.group)
        else:  # gloo has no reduce-scatter
            dist.all_reduce(xm, group=self.group)
            n = out.shape[0]
            out.copy_(xm[self.rank_in_group * n:(self.rank_in_group + 1) * n])
        return out.movedim(0, dim)

    def gather(self, x: torch.Tensor, dst: int = 0, dim: int = -1) -> Optional[torch.Tensor]:
        if self.world_size == 1:
            return x
        # all-gather then drop: keeps every rank on the same code path (graph friendly)
        out = self.all_gather(x, dim)
        return out if self.rank_in_group == dst else None

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(x, self.ranks[src], group=self.group)
        return x

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor, out_splits=None, in_splits=None):
        if self.world_size == 1:
            out.copy_(inp)
            return out
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)
        return out

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x.contiguous(), self.ranks[dst], group=self.group)

    def recv(self, shape, dtype, src: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, self.ranks[src], group=self.group)
        return t

    def isend_side_stream(self, x: torch.Tensor, dst: int):
        """Pipeline hand-off on a side stream so the next micro-batch's compute overlaps the copy."""
        if self._side_stream is None:
            return self.send(x, dst)
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._side_stream):
            self._side_stream.wait_event(ev)
            dist.send(x, self.ranks[dst], group=self.group)
            x.record_stream(self._side_stream)

    def barrier(self) -> None:
        if self.world_size > 1:
            if self.device.type == "cuda":
                dist.barrier(group=self.group, device_ids=[self.device.index or torch.cuda.current_device()])
            else:
                dist.barrier(group=self.group)

    @contextlib.contextmanager
    def change_state(self, disabled: bool):
        """Temporarily force the NCCL path (mirrors ``kunlun_communicator.py:66-86``)."""
        old = self.disabled
        self.disabled = disabled
        try:
            yield
        finally:
            self.disabled = old

    def destroy(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None
