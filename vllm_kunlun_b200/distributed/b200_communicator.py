"""``B200Communicator``: the device communicator upstream vLLM's ``GroupCoordinator`` instantiates for every
parallel group (TP / PP / EP / DP / DCP) on this platform.

Reference: ``KunlunCommunicator(CudaCommunicator)`` (``vllm_kunlun/distributed/kunlun_communicator.py:12-86``),
which turns every peer-memory fast path off (``ca_comm = None``, ``:28-32``) and sends each collective through the
library.  Here the constructor has the signature of the installed ``DeviceCommunicatorBase``; for tensor-parallel
groups on one node it maps every peer's symmetric buffers (:class:`vllm_kunlun_b200.parallel.symm_mem.PeerBuffers`)
and ``all_reduce`` of decode-sized payloads runs on the hand-written one-shot / low-latency NVLink kernels; larger
payloads, gathers and pipeline send / recv stay on ``torch.distributed`` (NCCL).  The warm-up all-reduce of the
reference (``:36-40``) doubles as the handshake after the peer-buffer exchange.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.distributed as dist

try:
    from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase
    HAVE_VLLM = True
except Exception:  # pragma: no cover
    DeviceCommunicatorBase = object  # type: ignore
    HAVE_VLLM = False


class B200Communicator(DeviceCommunicatorBase):
    def __init__(self, cpu_group, device: Optional[torch.device] = None, device_group=None, unique_name: str = "",
                 global_ranks: Optional[list] = None, global_world_size: Optional[int] = None):
        super().__init__(cpu_group, device, device_group, unique_name, global_ranks, global_world_size)
        self.disabled = False
        self.peer = None
        self.group = self.device_group  # the names the peer-buffer code reads
        kind = unique_name.split(":")[0]
        if (self.world_size > 1 and self.device.type == "cuda" and kind in ("tp", "ep", "")
                and self.world_size <= 8 and self.device_group is not None):
            try:
                from ..parallel.symm_mem import PeerBuffers
                self.peer = PeerBuffers.create(self)
            except Exception as e:  # peers not reachable (no NVLink / IPC): the library path serves everything
                import logging
                logging.getLogger(__name__).warning("peer-memory collectives unavailable for %s: %r", unique_name, e)
                self.peer = None
        if self.world_size > 1 and self.device_group is not None:
            t = torch.zeros(1, device=self.device)
            dist.all_reduce(t, group=self.device_group)  # warm-up / handshake

    # ---- collectives ----
    def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return input_
        if self.peer is not None and not self.disabled and self.peer.can_one_shot(input_):
            return self.peer.all_reduce(input_)
        return super().all_reduce(input_)

    def send(self, tensor: torch.Tensor, dst: Optional[int] = None) -> None:
        super().send(tensor, dst)

    def recv(self, size: torch.Size, dtype: torch.dtype, src: Optional[int] = None) -> torch.Tensor:
        return super().recv(size, dtype, src)

    @contextlib.contextmanager
    def change_state(self, disabled: bool):
        """Temporarily force the library path (the reference's ``change_state``, ``:66-86``)."""
        old, self.disabled = self.disabled, disabled
        try:
            yield
        finally:
            self.disabled = old

    def check_status(self) -> None:
        if self.peer is not None:
            self.peer.check_status()

    def destroy(self):
        if self.peer is not None:
            self.peer.close()
            self.peer = None
        if HAVE_VLLM:
            super().destroy()
