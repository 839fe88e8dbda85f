"""Expert-parallel token exchange: dispatch / combine over peer memory, and the library baseline.

Reference behaviour being replaced: with expert parallelism the reference keeps all tokens on all ranks, masks
per local expert in a Python loop and relies on the layer's all-reduce (call site C6,
``models/deepseek_v2.py:303-306``; ``KunlunOps.fused_moe_ep`` ``ops/_kunlun_ops.py:639-696``).

:class:`EPAll2All` serves layouts in which every rank holds its *own* tokens (sequence-parallel MoE,
``models/deepseek_v2.py:271-302``, or data-parallel attention): tokens travel once to each rank that owns one
of their top-k experts (fp8 + 1x128 scales for fp8 experts, bf16 otherwise), are processed by the grouped
GEMMs there, and the per-rank weighted partial sums travel back and are added in rank order.

:class:`EPLibraryBaseline` is the same computation with library collectives (all-gather the tokens and routing,
compute local experts on everything, reduce-scatter the partial sums); it runs on gloo as well, which is how the
multi-rank logic is tested without GPUs, and it is the comparison arm for the fused path on NVLink.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class EPAll2All:
    def __init__(self, comm, max_tokens_per_rank: int, hidden: int, topk: int, num_experts: int,
                 fp8_payload: bool = False, dtype=torch.bfloat16, spin_limit: int = 1 << 22):
        from ..ops import _ext
        C = self.C = _ext.C()
        self.comm, self.rank, self.R = comm, comm.rank_in_group, comm.world_size
        self.device = comm.device
        self.cap, self.H, self.k, self.E = int(max_tokens_per_rank), hidden, topk, num_experts
        self.fp8, self.dtype = fp8_payload, dtype
        assert num_experts % self.R == 0 and hidden % 128 == 0 and self.R <= 8
        self.row_bytes = hidden if fp8_payload else hidden * 2
        rows = self.R * self.cap
        o = {}
        cur = 0
        for name, nbytes in (("x", rows * self.row_bytes), ("scale", rows * (hidden // 128) * 4 if fp8_payload else 0),
                             ("ids", rows * topk * 4), ("w", rows * topk * 4), ("recv_flag", self.R * 8),
                             ("comb", rows * hidden * 2), ("comb_flag", self.R * 4)):
            o[name] = cur
            cur = _align(cur + nbytes)
        self.off, self.total = o, cur
        self.local = C.peer_alloc(self.total)
        dev = self.device.index or 0
        # ids of never-written rows must read as "no local expert"
        C.tensor_from_ptr(self.local + o["ids"], [rows * topk], torch.int32, dev).fill_(-1)
        torch.cuda.synchronize()
        handles = [None] * self.R
        use_cpu = comm.cpu_group is not None and dist.get_world_size() == self.R
        dist.all_gather_object(handles, C.peer_export(self.local), group=comm.cpu_group if use_cpu else comm.group)
        self.ptrs = [self.local if r == self.rank else C.peer_open(h) for r, h in enumerate(handles)]
        offs = [o[n] for n in ("x", "scale", "ids", "w", "recv_flag", "comb", "comb_flag")]
        self.h = C.EpHandle(self.ptrs, offs, self.rank, self.cap, hidden, topk, num_experts, self.row_bytes, self.cap,
                            spin_limit, dev)
        self.recv_x = C.tensor_from_ptr(self.local + o["x"], [rows, self.row_bytes], torch.uint8, dev)
        self.recv_scale = (C.tensor_from_ptr(self.local + o["scale"], [rows, hidden // 128], torch.float32, dev)
                           if fp8_payload else None)
        self.recv_ids = C.tensor_from_ptr(self.local + o["ids"], [rows, topk], torch.int32, dev)
        self.recv_w = C.tensor_from_ptr(self.local + o["w"], [rows, topk], torch.float32, dev)
        self.e_local = num_experts // self.R
        self._state = torch.zeros(2 * self.e_local, dtype=torch.int32, device=self.device)
        self.max_rows = 0  # bound on permuted rows per call; 0 = worst case (no token is ever dropped)
        torch.cuda.synchronize()
        dist.barrier(group=comm.group, device_ids=[dev])

    def check_status(self):
        s = int(self.h.status())
        if s:
            raise RuntimeError(f"expert-parallel exchange gave up waiting (code {s}: 41x slot overflow, 42x dispatch, "
                               "43x/44x combine; last digit = peer rank)")

    # ---- the three stages
    def _cap(self, bound: Optional[int]) -> int:
        """Per-call capacity of a source region: the largest token count any rank brings to this call, rounded up
        (every rank must pass the same bound); ``None`` = the allocated capacity."""
        if bound is None:
            return self.cap
        c = max(8, (int(bound) + 7) // 8 * 8)
        assert c <= self.cap, f"{bound} tokens per rank exceed the allocated capacity {self.cap}"
        return c

    def dispatch(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, bound: Optional[int] = None):
        cap = self._cap(bound)
        assert x.shape[0] <= cap
        if self.fp8:
            if x.shape[0]:
                q, st = self.C.quant_fp8_group(x, False, None, 4)
            else:
                q = torch.empty(0, self.H, dtype=torch.uint8, device=self.device)
                st = torch.zeros(self.H // 128, 4, dtype=torch.float32, device=self.device)
            self.h.dispatch(q, st, topk_ids.int().contiguous(), topk_w.float().contiguous(), cap)
        else:
            self.h.dispatch(x, None, topk_ids.int().contiguous(), topk_w.float().contiguous(), cap)

    def experts(self, w13, w2, act="silu", b13=None, b2=None, w13_scale=None, w2_scale=None, bound: Optional[int] = None):
        """Grouped GEMMs over the received rows; returns ``(y_sorted, pos_of_pair)``."""
        C = self.C
        E = self.e_local
        rows = self.R * self._cap(bound)
        recv_x, recv_ids = self.recv_x[:rows], self.recv_ids[:rows]
        if self.fp8:
            xs, pos, lod = C.moe_permute(recv_x.view(torch.bfloat16), recv_ids, None, E, E, self._state, self.max_rows)
            M = xs.shape[0]
            q = xs.view(torch.uint8)
            stride = max(4, (M + 3) // 4 * 4)
            st = torch.zeros(self.H // 128, stride, dtype=torch.float32, device=self.device)
            self.h.permute_scales(st, self.recv_scale[:rows], pos)
            h = torch.empty(M, w13.shape[1], dtype=self.dtype, device=self.device)
            C.grouped_gemm(h, q, w13.view(torch.uint8), lod, b13, st, w13_scale, 0)
            a = ops.act_and_mul(h, act)
            q2, st2 = C.quant_fp8_group(a, False, lod[E:], 4)
            y = torch.empty(M, self.H, dtype=self.dtype, device=self.device)
            C.grouped_gemm(y, q2, w2.view(torch.uint8), lod, b2, st2, w2_scale, 0)
        else:
            xs, pos, lod = C.moe_permute(recv_x.view(self.dtype), recv_ids, None, E, E, self._state, self.max_rows)
            M = xs.shape[0]
            h = torch.empty(M, w13.shape[1], dtype=self.dtype, device=self.device)
            C.grouped_gemm(h, xs, w13, lod, b13, None, None, 0)
            a = ops.act_and_mul(h, act)
            y = torch.empty(M, self.H, dtype=self.dtype, device=self.device)
            C.grouped_gemm(y, a, w2, lod, b2, None, None, 0)
        return y, pos

    def combine(self, y_sorted, pos, num_tokens: int, addend: Optional[torch.Tensor] = None, bound: Optional[int] = None):
        out = torch.empty(num_tokens, self.H, dtype=self.dtype, device=self.device)
        self.h.combine(y_sorted, pos, out, addend, self._cap(bound))
        return out

    def moe(self, x, topk_ids, topk_w, w13, w2, act="silu", b13=None, b2=None, w13_scale=None, w2_scale=None, addend=None,
            bound: Optional[int] = None):
        self.dispatch(x, topk_ids, topk_w, bound)
        y, pos = self.experts(w13, w2, act, b13, b2, w13_scale, w2_scale, bound)
        return self.combine(y, pos, x.shape[0], addend, bound)


class EPLibraryBaseline:
    """All-gather tokens + routing, local experts over everything, reduce-scatter (NCCL or gloo)."""

    def __init__(self, group, rank: int, world: int, num_experts: int):
        self.group, self.rank, self.R, self.E = group, rank, world, num_experts
        self.e_local = num_experts // world
        emap = torch.full((num_experts,), -1, dtype=torch.int32)
        emap[rank * self.e_local:(rank + 1) * self.e_local] = torch.arange(self.e_local, dtype=torch.int32)
        self.emap = emap

    def moe(self, x, topk_ids, topk_w, w13, w2, act="silu", b13=None, b2=None, w13_scale=None, w2_scale=None, addend=None):
        """Every rank passes the same number of tokens."""
        R, T = self.R, x.shape[0]
        xs = torch.empty(R * T, x.shape[1], dtype=x.dtype, device=x.device)
        ids = torch.empty(R * T, topk_ids.shape[1], dtype=torch.int32, device=x.device)
        ws = torch.empty(R * T, topk_w.shape[1], dtype=torch.float32, device=x.device)
        dist.all_gather_into_tensor(xs, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(ids, topk_ids.int().contiguous(), group=self.group)
        dist.all_gather_into_tensor(ws, topk_w.float().contiguous(), group=self.group)
        part = ops.fused_moe(xs, w13, w2, ws, ids, act, b13, b2, w13_scale, w2_scale, (128, 128), self.emap.to(x.device))
        if part.is_cuda:
            out = torch.empty(T, x.shape[1], dtype=part.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, part.contiguous(), group=self.group)
        else:  # gloo has no reduce-scatter
            dist.all_reduce(part, group=self.group)
            out = part[self.rank * T:(self.rank + 1) * T].clone()
        return out if addend is None else out + addend
