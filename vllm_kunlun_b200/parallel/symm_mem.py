"""Symmetric peer-memory buffers over NVLink / NVSwitch and the collectives built on them.

The reference communicator disables every peer-memory fast path (``ca_comm = None``,
``vllm_kunlun/distributed/kunlun_communicator.py:28-32``) and sends each row-parallel output through
a library all-reduce (call sites C1 / C2 / C4).  Here each rank of a group maps every peer's buffer
(CUDA IPC handles exchanged once over the process group) and hand-written kernels read and write
them directly: a one-shot all-reduce fused with the residual add and RMSNorm that follow it, and the
staging areas of the fused GEMM+collective kernels.

All cross-GPU waits are bounded and report through a status word; nothing here uses NVLS multicast.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _ext


class PeerBuffers:
    def __init__(self, comm, parity_bytes: int):
        self.comm = comm
        self.rank = comm.rank_in_group
        self.world = comm.world_size
        self.device = comm.device
        C = _ext.C()
        self.C = C
        self.parity_bytes = int(parity_bytes)
        self.flags_offset = 2 * self.parity_bytes
        self.total_bytes = self.flags_offset + C.allreduce_flag_bytes()
        self.local_ptr = C.peer_alloc(self.total_bytes)
        handle = C.peer_export(self.local_ptr)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=comm.cpu_group if self._use_cpu_group() else comm.group)
        self.ptrs = []
        for r, h in enumerate(handles):
            self.ptrs.append(self.local_ptr if r == self.rank else C.peer_open(h))
        self.epochs = torch.zeros(C.allreduce_max_ctas(), dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.max_ctas = C.allreduce_max_ctas()
        self.spin_limit = 1 << 22
        self.one_shot_max_bytes = min(self.parity_bytes, 2 << 20)
        self.launches = 0
        torch.cuda.synchronize()
        dist.barrier(group=comm.group, device_ids=[self.device.index or 0])

    def _use_cpu_group(self) -> bool:
        # the cpu (gloo) group spans the whole world; only usable when this group is the world
        return self.comm.cpu_group is not None and dist.get_world_size() == self.world

    @classmethod
    def create(cls, comm, parity_bytes: int = 8 << 20) -> Optional["PeerBuffers"]:
        if not _ext.available() or comm.device.type != "cuda":
            return None
        return cls(comm, parity_bytes)

    # ------------------------------------------------------------------ collectives
    def can_one_shot(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dim() >= 1 and x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
                and x.numel() * x.element_size() <= self.one_shot_max_bytes
                and (x.shape[-1] * x.element_size()) % 16 == 0)

    def _grid(self, rows: int) -> int:
        return max(1, min(rows, self.max_ctas))

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        out = torch.empty_like(x2) if out is None else out.reshape(-1, x.shape[-1])
        self.C.oneshot_allreduce(self.ptrs, x2, out, None, None, self.epochs, self.status, self.parity_bytes,
                                 self.flags_offset, self.rank, 0.0, False, self._grid(x2.shape[0]), self.spin_limit)
        self.launches += 1
        return out.reshape(x.shape)

    def all_reduce_add_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                               gemma: bool = False):
        """``residual += all_reduce(x); x = rmsnorm(residual) * w`` in one kernel; returns ``(x, residual)``."""
        x2 = x.reshape(-1, x.shape[-1])
        self.C.oneshot_allreduce(self.ptrs, x2, x2, residual.reshape(-1, x.shape[-1]), weight, self.epochs,
                                 self.status, self.parity_bytes, self.flags_offset, self.rank, eps, gemma,
                                 self._grid(x2.shape[0]), self.spin_limit)
        self.launches += 1
        return x, residual

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"peer all-reduce: bounded wait on rank {code - 200} timed out")

    def close(self) -> None:
        if self.local_ptr is None:
            return
        torch.cuda.synchronize()
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.C.peer_close(p)
        try:
            dist.barrier(group=self.comm.group, device_ids=[self.device.index or 0])
        except Exception:
            pass
        self.C.peer_free(self.local_ptr)
        self.local_ptr = None
