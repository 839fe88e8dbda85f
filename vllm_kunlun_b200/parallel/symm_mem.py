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

import os

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
        # low-latency buffers for decode-sized payloads: 2 parities x world slots, payload + flags interleaved
        import os
        self.ll_max_bytes = 256 << 10 if os.environ.get("B200_AR_LL", "1") != "0" else 0
        self.ll_slot_bytes = 2 * self.ll_max_bytes
        self.ll_ptrs = None
        if self.ll_max_bytes:
            self.ll_local = C.peer_alloc(2 * self.world * self.ll_slot_bytes)
            ll_handles = [None] * self.world
            dist.all_gather_object(ll_handles, C.peer_export(self.ll_local),
                                   group=comm.cpu_group if self._use_cpu_group() else comm.group)
            self.ll_ptrs = [self.ll_local if r == self.rank else C.peer_open(h) for r, h in enumerate(ll_handles)]
            self.ll_epochs = torch.zeros(C.allreduce_max_ctas(), dtype=torch.int32, device=self.device)
        self.epochs = torch.zeros(C.allreduce_max_ctas(), dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.max_ctas = C.allreduce_max_ctas()
        # polls before a wait on a peer gives up (about 10 s): long enough for a peer that is still capturing a
        # CUDA graph or loading a module; failure-detection tests pass their own small limit
        self.spin_limit = int(os.environ.get("B200_PEER_SPIN_LIMIT", str(1 << 26)))
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

    def _can_ll(self, x2: torch.Tensor) -> bool:
        return (self.ll_ptrs is not None and x2.element_size() == 2 and x2.shape[-1] % 8 == 0
                and x2.numel() * 2 <= self.ll_max_bytes)

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        out = torch.empty_like(x2) if out is None else out.reshape(-1, x.shape[-1])
        if self._can_ll(x2):
            self.C.ll_allreduce(self.ll_ptrs, x2, out, None, None, self.ll_epochs, self.status, self.ll_slot_bytes,
                                self.rank, 0.0, False, self._grid(x2.shape[0]), self.spin_limit, False)
            self.launches += 1
            return out.reshape(x.shape)
        self.C.oneshot_allreduce(self.ptrs, x2, out, None, None, self.epochs, self.status, self.parity_bytes,
                                 self.flags_offset, self.rank, 0.0, False, self._grid(x2.shape[0]), self.spin_limit)
        self.launches += 1
        return out.reshape(x.shape)

    def can_push(self, rows: int, width: int, dtype) -> bool:
        """Whether a row-parallel decode GEMM of this output shape may push its partials from the epilogue."""
        return (self.ll_ptrs is not None and rows <= 32 and width % 128 == 0 and dtype in (torch.bfloat16, torch.float16)
                and rows * width * 2 <= self.ll_max_bytes)

    def all_reduce_add_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                               gemma: bool = False, pushed: bool = False):
        """``residual += all_reduce(x); x = rmsnorm(residual) * w`` in one kernel; returns ``(x, residual)``.
        ``pushed``: the GEMM that produced ``x`` has already written it into the peers' slots."""
        x2 = x.reshape(-1, x.shape[-1])
        if self._can_ll(x2):
            self.C.ll_allreduce(self.ll_ptrs, x2, x2, residual.reshape(-1, x.shape[-1]), weight, self.ll_epochs,
                                self.status, self.ll_slot_bytes, self.rank, eps, gemma, self._grid(x2.shape[0]),
                                self.spin_limit, pushed)
            self.launches += 1
            return x, residual
        assert not pushed
        self.C.oneshot_allreduce(self.ptrs, x2, x2, residual.reshape(-1, x.shape[-1]), weight, self.epochs,
                                 self.status, self.parity_bytes, self.flags_offset, self.rank, eps, gemma,
                                 self._grid(x2.shape[0]), self.spin_limit)
        self.launches += 1
        return x, residual

    # ------------------------------------------------------------------ fused GEMM + collectives
    # Sequence-parallel chain for large token counts (prefill), all over peer memory:
    #   row-parallel GEMM  --(epilogue stores tiles into the owner rank's staging area)-->  reduce-scatter
    #   rs_norm_ag kernel  --(sum + residual + RMSNorm, rows pushed to every rank)-------->  all-gather
    #   column-parallel GEMM (TMA producer waits per token tile for the pushed rows)
    # Two call parities alternate.  Counters of parity p are zeroed by the rs_norm_ag kernel of the next
    # call (parity 1-p): by then this rank's consumers of parity p have finished (stream order), and no
    # peer can produce for parity p again before it has consumed this rank's pushes of that next call.
    SP_MAX_TT = 512

    def sp_init(self, max_tokens: int, hidden: int, dtype=torch.bfloat16) -> None:
        if getattr(self, "sp_ready", False):
            return
        C = self.C
        es = torch.empty((), dtype=dtype).element_size()
        self.sp_H, self.sp_T, self.sp_dtype = hidden, max_tokens, dtype
        self.sp_stage_off = 0
        self.sp_xfull_off = max_tokens * hidden * es
        self.sp_rsflag_off = 2 * max_tokens * hidden * es
        self.sp_agflag_off = self.sp_rsflag_off + 2 * self.world * self.SP_MAX_TT * 4
        total = self.sp_agflag_off + 2 * self.SP_MAX_TT * 4
        self.sp_local = C.peer_alloc(total)
        handles = [None] * self.world
        dist.all_gather_object(handles, C.peer_export(self.sp_local),
                               group=self.comm.cpu_group if self._use_cpu_group() else self.comm.group)
        self.sp_ptrs = [self.sp_local if r == self.rank else C.peer_open(h) for r, h in enumerate(handles)]
        self.sp_calls = 0
        self.sp_pending = None
        self.sp_ready = True
        torch.cuda.synchronize()
        dist.barrier(group=self.comm.group, device_ids=[self.device.index or 0])

    def sp_ok(self, T: int, hidden: int, dtype) -> bool:
        if not getattr(self, "sp_ready", False):
            return False
        R = self.world
        return (dtype == self.sp_dtype and hidden == self.sp_H and T <= self.sp_T and T % (R * 64) == 0
                and T // 64 <= self.SP_MAX_TT and hidden % 128 == 0)

    @staticmethod
    def _pick_bn(n: int) -> int:
        for bn in (256, 128, 64):
            if n % bn == 0:
                return bn
        raise ValueError(n)

    def _rs_flags(self, r: int, parity: int) -> int:
        return self.sp_ptrs[r] + self.sp_rsflag_off + parity * self.world * self.SP_MAX_TT * 4

    def _ag_flags(self, r: int, parity: int) -> int:
        return self.sp_ptrs[r] + self.sp_agflag_off + parity * self.SP_MAX_TT * 4

    def gemm_rs(self, x: torch.Tensor, weight: torch.Tensor):
        """Row-parallel partial GEMM whose epilogue scatters the tiles to the token owners.
        Returns a handle for :meth:`rs_norm_ag`."""
        from ..ops import gemm_cuda
        T, R = x.shape[0], self.world
        tloc = T // R
        bn = self._pick_bn(tloc)
        parity = self.sp_calls & 1
        self.sp_calls += 1
        stage = [p + self.sp_stage_off for p in self.sp_ptrs]
        flags = [self._rs_flags(r, parity) + self.rank * self.SP_MAX_TT * 4 for r in range(R)]
        self.C.set_gemm_comm(stage, flags, 0, tloc, self.rank, 0)
        gemm_cuda.gemm_bf16(x, weight, None, out=self._fake_out(T, weight.shape[0], x), splits=1, bn=bn)
        self.launches += 1
        return {"T": T, "tloc": tloc, "bn": bn, "parity": parity, "N": weight.shape[0]}

    def _fake_out(self, T, N, x):
        # the GEMM API wants an output tensor of the right shape; in reduce-scatter mode nothing is
        # written to it, so a view of the (large enough) local staging area serves
        return self.C.tensor_from_ptr(self.sp_local + self.sp_stage_off, [T, N], x.dtype, self.device.index or 0)

    def rs_norm_ag(self, handle, residual, weight, eps: float, gemma: bool = False):
        """Reduce the scattered partials, add the residual (own rows), RMSNorm, gather to all ranks.
        Returns the gathered activations ``[T, H]`` (a view of this rank's symmetric buffer); the next
        GEMM on that tensor waits per token tile for the rows to arrive."""
        T, tloc, bn, parity = handle["T"], handle["tloc"], handle["bn"], handle["parity"]
        R, H = self.world, self.sp_H
        ag_bn = self._pick_bn(T) if T % 64 == 0 else 64
        prev = 1 - parity
        self.C.rs_norm_ag(self.sp_local + self.sp_stage_off, self._rs_flags(self.rank, parity),
                          [p + self.sp_xfull_off for p in self.sp_ptrs], [self._ag_flags(r, parity) for r in range(R)],
                          self._rs_flags(self.rank, prev), R * self.SP_MAX_TT, self._ag_flags(self.rank, prev),
                          self.SP_MAX_TT, residual, weight, self.status, self.rank, tloc, H, bn, H // 128, ag_bn, 4,
                          self.SP_MAX_TT, eps, gemma, self.spin_limit)
        self.launches += 1
        x = self.C.tensor_from_ptr(self.sp_local + self.sp_xfull_off, [T, H], self.sp_dtype, self.device.index or 0)
        self.sp_pending = {"ptr": x.data_ptr(), "flags": self._ag_flags(self.rank, parity), "expect": ag_bn,
                           "bn": ag_bn, "n_tt": T // ag_bn}
        return x

    def sp_consume(self, x: torch.Tensor):
        """Called by the GEMM entry: if ``x`` is the pending gathered buffer, arm the all-gather wait
        for the next GEMM launch and return its token tile size."""
        pd = getattr(self, "sp_pending", None)
        if pd is None or x.data_ptr() != pd["ptr"]:
            return 0
        self.C.set_gemm_comm([], [], pd["flags"], 0, self.rank, pd["expect"])
        self.sp_pending = None
        return pd["bn"]

    def sp_sync(self) -> None:
        """Make the stream wait for all gathered rows (for consumers other than the fused GEMM)."""
        pd = getattr(self, "sp_pending", None)
        if pd is not None:
            self.C.sp_wait(pd["flags"], pd["n_tt"], pd["expect"], self.spin_limit, self.status)
            self.sp_pending = None

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"peer-memory collective: a bounded wait timed out (code {code})")

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
        if getattr(self, "sp_ready", False):
            for r, p in enumerate(self.sp_ptrs):
                if r != self.rank:
                    self.C.peer_close(p)
            self.C.peer_free(self.sp_local)
            self.sp_ready = False
