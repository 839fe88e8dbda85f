"""Tensor-parallel building blocks: linears, embedding, norms, rotary caches.

Parity targets in the reference: ``ops/linear.py`` (merged-column / QKV weight loaders with
block-scale shard arithmetic ``:91-96``), ``ops/vocab_parallel_embedding.py:94-118``,
``ops/layernorm.py:71-167`` and ``ops/rotary_embedding/*``.  Weight tensors keep the checkpoint
layout ``[out_features, in_features]``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from .. import ops
from ..config import cdiv
from ..parallel.state import get_state

DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
          "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16, "torch.float32": torch.float32}


def param(*shape, dtype, device) -> nn.Parameter:
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)


# --------------------------------------------------------------------------- quant method plumbing

class UnquantizedLinearMethod:
    """bf16 / fp16 / fp32 weights, GEMM through :func:`ops.linear` (tcgen05 on CUDA)."""

    name = None

    def create_weights(self, layer: "LinearBase", out_local: int, in_local: int, dtype, device):
        layer.weight = param(out_local, in_local, dtype=dtype, device=device)

    def apply(self, layer: "LinearBase", x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, layer.weight, layer.bias)

    def process_weights_after_loading(self, layer):
        pass

    # rows/cols of every quant-aux tensor that shard with the weight: name -> (row_div, col_div)
    def aux_params(self):
        return {}


_QUANT_METHODS = {None: UnquantizedLinearMethod}


def register_linear_method(name: str, cls) -> None:
    _QUANT_METHODS[name] = cls


_QUANT_DEFAULTS: dict = {}   # method name -> constructor arguments taken from the checkpoint's quantization_config


def set_quant_defaults(name: Optional[str], kw: Optional[dict]) -> None:
    """Arguments (group size, bits, ...) for the layers of the model about to be built (``build_model``)."""
    if name:
        _QUANT_DEFAULTS[name] = dict(kw or {})


def get_linear_method(name: Optional[str], **kw):
    if name not in _QUANT_METHODS:
        from .. import quantization  # noqa: F401  (registers the methods)
    if not kw and name in _QUANT_DEFAULTS:
        kw = _QUANT_DEFAULTS[name]
    return _QUANT_METHODS[name](**kw)


def _kn_spec(method, name: str):
    """``(k_div, n_div)`` of an input-major checkpoint tensor ``[K / k_div, N / n_div]`` (AWQ / GPTQ ``qweight``,
    ``qzeros``, ``scales``; ``g_idx [K]`` has ``n_div`` None), else None."""
    fn = getattr(method, "kn_params", None)
    return fn().get(name) if fn is not None else None


class LinearBase(nn.Module):
    def __init__(self, in_features, out_features, bias, dtype, device, quant: Optional[str], quant_kw=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.method = get_linear_method(quant, **(quant_kw or {}))
        self.bias = None
        self._dtype, self._device = dtype, device

    def forward(self, x):
        return self.method.apply(self, x)


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, device="cpu", quant=None,
                 quant_kw=None):
        super().__init__(in_features, out_features, bias, dtype, device, quant, quant_kw)
        self.method.create_weights(self, out_features, in_features, dtype, device)
        if bias:
            self.bias = param(out_features, dtype=dtype, device=device)

    def load(self, name: str, w: torch.Tensor, shard_id=None):
        getattr(self, name).data.copy_(w)


class ColumnParallelLinear(LinearBase):
    """Output dimension sharded over TP.  ``output_sizes`` lists the logical partitions of a merged
    projection (e.g. ``[q, k, v]`` or ``[gate, up]``); each is sharded separately so a rank holds the
    matching slices of all of them (``MergedColumnParallelLinear`` / ``QKVParallelLinear``)."""

    def __init__(self, in_features, output_sizes: Sequence[int], bias=False, dtype=torch.bfloat16,
                 device="cpu", quant=None, tp_size=None, tp_rank=None, replicate: Sequence[bool] = (),
                 quant_kw=None):
        st = get_state()
        self.tp_size = st.tp_size if tp_size is None else tp_size
        self.tp_rank = st.tp_rank if tp_rank is None else tp_rank
        self.output_sizes = list(output_sizes)
        # a partition marked "replicate" is kept whole on every rank (KV heads when tp > kv_heads)
        self.replicate = list(replicate) or [False] * len(self.output_sizes)
        self.local_sizes = [s if r else s // self.tp_size for s, r in zip(self.output_sizes, self.replicate)]
        super().__init__(in_features, sum(self.output_sizes), bias, dtype, device, quant, quant_kw)
        self.out_local = sum(self.local_sizes)
        self.method.create_weights(self, self.out_local, in_features, dtype, device)
        if bias:
            self.bias = param(self.out_local, dtype=dtype, device=device)

    def _shard_rows(self, shard_id: Optional[int], row_div: int = 1):
        """(dst_start, dst_len, src_start) in units of ``row_div`` rows for partition ``shard_id``."""
        ids = range(len(self.output_sizes)) if shard_id is None else [shard_id]
        out = []
        for i in ids:
            dst0 = sum(self.local_sizes[:i])
            ln = self.local_sizes[i]
            src0 = 0 if self.replicate[i] else self.tp_rank * ln
            # block-scale tensors: ceil-divide, as ``adjust_block_scale_shard`` does (ops/linear.py:91-96)
            out.append((cdiv(dst0, row_div) if row_div > 1 else dst0,
                        cdiv(ln, row_div) if row_div > 1 else ln,
                        src0 // row_div, i))
        return out

    def _load_kn(self, name: str, w: torch.Tensor, shard_id: Optional[int], kn, kv_head_shard=None):
        """Input-major tensor ``[K / k_div, N / n_div]``: the output partitions lie along dim 1."""
        p = getattr(self, name)
        n_div = kn[1]
        if n_div is None:               # per-input vector (g_idx): the same on every rank
            p.data.copy_(w.reshape(p.shape))
            return
        if shard_id is None and len(self.output_sizes) > 1:
            offs = 0
            for i, s in enumerate(self.output_sizes):
                self._load_kn(name, w[:, offs // n_div:(offs + s) // n_div], i, kn, kv_head_shard)
                offs += s
            return
        for dst0, ln, src0, i in self._shard_rows(shard_id if shard_id is not None else 0):
            if kv_head_shard is not None and self.replicate[i]:
                src0 = kv_head_shard(i)
            assert dst0 % n_div == 0 and ln % n_div == 0 and src0 % n_div == 0, \
                f"{name}: partition of {ln} columns at {src0} does not fall on the packing of {n_div}"
            p.data[:, dst0 // n_div:(dst0 + ln) // n_div].copy_(w[:, src0 // n_div:(src0 + ln) // n_div])

    def load(self, name: str, w: torch.Tensor, shard_id: Optional[int] = None, kv_head_shard=None):
        p = getattr(self, name)
        kn = _kn_spec(self.method, name)
        if kn is not None:
            return self._load_kn(name, w, shard_id, kn, kv_head_shard)
        aux = self.method.aux_params().get(name)
        row_div = aux[0] if aux else 1
        if shard_id is None and len(self.output_sizes) > 1:
            # fused checkpoint tensor: split along rows by logical partition first
            offs = 0
            for i, s in enumerate(self.output_sizes):
                n = cdiv(s, row_div)
                self.load(name, w[offs:offs + n], i)
                offs += n
            return
        for dst0, ln, src0, i in self._shard_rows(shard_id if shard_id is not None else 0, row_div):
            if kv_head_shard is not None and self.replicate[i]:
                src0 = kv_head_shard(i) // row_div
            if p.dim() == 0:
                p.data.copy_(w.reshape(()))
            else:
                p.data[dst0:dst0 + ln].copy_(w[src0:src0 + ln])


class RowParallelLinear(LinearBase):
    """Input dimension sharded over TP; partial sums are combined by all-reduce
    (call site C1/C2 of the reference: ``models/deepseek_v2.py:126-134,399-405``) unless
    ``reduce_results`` is False (the caller fuses the reduction)."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, device="cpu",
                 quant=None, reduce_results=True, tp_size=None, tp_rank=None, quant_kw=None):
        st = get_state()
        self.tp_size = st.tp_size if tp_size is None else tp_size
        self.tp_rank = st.tp_rank if tp_rank is None else tp_rank
        super().__init__(in_features, out_features, bias, dtype, device, quant, quant_kw)
        self.in_local = in_features // self.tp_size
        self.reduce_results = reduce_results
        # set by the owner when the output goes straight into reduce_add_rmsnorm: decode-sized calls then push
        # their partial sums to the peers from the GEMM epilogue
        self.push_ok = False
        self.method.create_weights(self, out_features, self.in_local, dtype, device)
        if bias:
            self.bias = param(out_features, dtype=dtype, device=device)

    def forward(self, x):
        if (self.tp_size > 1 and not self.reduce_results and self.bias is None and x.is_cuda
                and type(self.method) is UnquantizedLinearMethod):
            peer = getattr(get_state().tp_comm, "peer", None)
            if peer is not None and sp_mode_active() and peer.sp_ok(x.shape[0], self.out_features, x.dtype):
                # GEMM -> reduce-scatter fused over peer memory; finished by reduce_add_rmsnorm
                return SPPartial(peer, peer.gemm_rs(x.reshape(-1, x.shape[-1]), self.weight))
            if (peer is not None and self.push_ok and PUSH_EPILOGUE[0] and x.dim() == 2 and not get_state().tp_comm.disabled
                    and peer.can_push(x.shape[0], self.out_features, x.dtype)):
                from ..ops.gemm_cuda import gemm_decode_push
                y = gemm_decode_push(x, self.weight, peer)
                y._b200_pushed = peer  # the consumer (reduce_add_rmsnorm) only collects
                return y
        bias = self.bias
        if self.tp_rank != 0:
            self.bias = None  # add the bias once
        try:
            y = self.method.apply(self, x)
        finally:
            self.bias = bias
        if self.reduce_results and self.tp_size > 1:
            y = get_state().tp_comm.all_reduce(y)
        return y

    def load(self, name: str, w: torch.Tensor, shard_id=None):
        p = getattr(self, name)
        kn = _kn_spec(self.method, name)
        if kn is not None:      # input-major tensor [K / k_div, ...]: this rank's inputs are a block of rows
            k_div = kn[0]
            assert (self.tp_rank * self.in_local) % k_div == 0 and self.in_local % k_div == 0, \
                f"{name}: {self.in_local} inputs per rank do not fall on the packing / group size of {k_div}"
            r0 = (self.tp_rank * self.in_local) // k_div
            rows = w[r0:r0 + self.in_local // k_div]
            if kn[1] is None:   # g_idx: group numbers restart at this rank's first group
                rows = rows - (rows.min() if rows.numel() else 0)
            p.data.copy_(rows.reshape(p.shape))
            return
        if name == "bias" or p.dim() < 2:
            p.data.copy_(w.reshape(p.shape))
            return
        if w.dim() == 2 and w.shape[1] == 1 and p.shape[1] == 1:
            p.data.copy_(w)     # one value per output channel (int8 weight scales): the same on every rank
            return
        aux = self.method.aux_params().get(name)
        col_div = aux[1] if aux else 1
        n = p.shape[1]
        s0 = (self.tp_rank * self.in_local) // col_div
        p.data.copy_(w[:, s0:s0 + n])


class VocabParallelEmbedding(nn.Module):
    """Rows sharded over TP; lookups outside the shard give zeros, then all-reduce (C4)."""

    def __init__(self, vocab_size, hidden, dtype=torch.bfloat16, device="cpu", pad_to: int = 64):
        super().__init__()
        st = get_state()
        self.tp_size, self.tp_rank = st.tp_size, st.tp_rank
        self.vocab_size = vocab_size
        self.padded = cdiv(vocab_size, pad_to * self.tp_size) * pad_to * self.tp_size
        self.rows = self.padded // self.tp_size
        self.start = self.tp_rank * self.rows
        self.weight = param(self.rows, hidden, dtype=dtype, device=device)

    def forward(self, ids):
        out = ops.embedding(ids, self.weight, self.start)
        if self.tp_size > 1:
            out = get_state().tp_comm.all_reduce(out)
        return out

    def load(self, name, w, shard_id=None):
        n = max(0, min(self.rows, w.shape[0] - self.start))
        self.weight.data.zero_()
        if n > 0:
            self.weight.data[:n].copy_(w[self.start:self.start + n])


class ParallelLMHead(VocabParallelEmbedding):
    """Logits = hidden @ W.T on the local vocab shard, then all-gather (C5)."""

    def logits(self, hidden, weight=None):
        w = self.weight if weight is None else weight
        lg = ops.linear(hidden, w)
        if self.tp_size > 1:
            lg = get_state().tp_comm.all_gather(lg, dim=-1)
        return lg[..., : self.vocab_size]


class RMSNorm(nn.Module):
    def __init__(self, size, eps, dtype=torch.bfloat16, device="cpu", gemma=False):
        super().__init__()
        self.weight = param(size, dtype=dtype, device=device)
        self.eps, self.gemma = eps, gemma

    def forward(self, x, residual=None):
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps, self.gemma)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, self.gemma)

    def load(self, name, w, shard_id=None):
        self.weight.data.copy_(w)


class SPPartial:
    """Result of a row-parallel GEMM whose tiles were scattered to their owner ranks."""

    def __init__(self, peer, handle):
        self.peer, self.handle = peer, handle


_SP_MODE = False
import os as _os
PUSH_EPILOGUE = [_os.environ.get("B200_GEMM_PUSH", "1") != "0"]


def sp_mode_active() -> bool:
    return _SP_MODE


def set_sp_mode(on: bool) -> None:
    """Enabled by the runner for eager steps (never while capturing a CUDA graph)."""
    global _SP_MODE
    _SP_MODE = on


def sp_sync():
    """Wait for gathered activations before a consumer that is not the fused GEMM."""
    st = get_state()
    peer = getattr(st.tp_comm, "peer", None) if st.tp_comm is not None else None
    if peer is not None and getattr(peer, "sp_pending", None) is not None:
        peer.sp_sync()


def reduce_add_rmsnorm(x, residual, norm: "RMSNorm", partial: bool):
    """``residual += all_reduce(x); out = norm(residual)`` for a row-parallel partial ``x``.

    With mapped peer memory and a decode-sized payload this is ONE kernel (peer loads + add + norm,
    replacing all-reduce call sites C1 / C2 of the reference plus the ``add_rmsnorm`` that follows
    them); otherwise a collective followed by the fused add+norm kernel."""
    st = get_state()
    if isinstance(x, SPPartial):
        out = x.peer.rs_norm_ag(x.handle, residual, norm.weight, norm.eps, norm.gemma)
        return out, residual
    if partial and st.tp_size > 1:
        comm = st.tp_comm
        if (residual is not None and comm.peer is not None and not comm.disabled
                and comm.peer.can_one_shot(x)):
            pushed = getattr(x, "_b200_pushed", None) is comm.peer
            return comm.peer.all_reduce_add_rmsnorm(x, residual, norm.weight, norm.eps, norm.gemma, pushed=pushed)
        x = comm.all_reduce(x)
    if residual is None:
        return norm(x), x
    return norm(x, residual)


_ROPE_CACHE: dict = {}


def get_cos_sin_cache(rotary_dim, max_pos, theta, scaling, device) -> torch.Tensor:
    """Process-wide cache of cos/sin tables (``get_rope`` registry, ``ops/rotary_embedding/rope_ext.py:67-108``)."""
    key = (rotary_dim, max_pos, theta, None if scaling is None else tuple(vars(scaling).items()), str(device))
    if key not in _ROPE_CACHE:
        from ..ops.reference.basic import build_cos_sin_cache
        _ROPE_CACHE[key] = build_cos_sin_cache(rotary_dim, max_pos, theta, scaling).to(device)
    return _ROPE_CACHE[key]
