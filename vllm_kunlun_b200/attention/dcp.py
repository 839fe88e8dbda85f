"""Decode context parallelism for MLA: the latent KV cache of a sequence is interleaved over the ranks of the
DCP group (token ``p`` lives on rank ``p % dcp`` at local position ``p // dcp``), so every rank holds and reads
``1 / dcp`` of the context.

Reference: ``v1/attention/backends/mla/common.py`` - per-rank local lengths of the interleaved cache (:517-557), decode ``q`` all-gathered along the head dimension (:2030-2035), local attention returning the LSE,
``cp_lse_ag_out_rs`` = LSE all-gather + output correction + reduce-scatter over heads (:2044); the prefill
context takes another route there (``cp_gather_cache`` + all-gather + ``reorg_kvcache``, :1679-1780, :922-990).

Here one routine serves every step.  Each query token becomes its own row with its own local context length
``(pos - rank) // dcp + 1``, which makes the causal mask exact for prefill chunks as well, so no K/V ever crosses
the link: only queries (all-gather), log-sum-exps (all-gather) and corrected outputs (reduce-scatter)."""
from __future__ import annotations

import torch

from .. import ops


def local_context_len(positions: torch.Tensor, dcp: int, rank: int) -> torch.Tensor:
    """Number of cached tokens on ``rank`` visible to a query at global position ``positions`` (inclusive)."""
    return torch.clamp(torch.div(positions - rank, dcp, rounding_mode="floor") + 1, min=0)


def dcp_slot(position: int, block_ids, block_size: int, dcp: int, rank: int) -> int:
    """Cache slot of a token on this rank, or -1 when another rank owns it.  A block of the block table covers
    ``block_size * dcp`` consecutive tokens of the sequence, ``block_size`` of them on each rank."""
    if position % dcp != rank:
        return -1
    vb = block_size * dcp
    return block_ids[position // vb] * block_size + (position % vb) // dcp


def dcp_mla_attention(q, kv_cache, md, scale: float, kv_lora_rank: int, st):
    """``q [T, N_local, 576]`` -> ``out [T, N_local, kv_lora_rank]`` with the context spread over ``st.dcp_comm``."""
    dcp, rank, comm = st.dcp_size, st.dcp_rank, st.dcp_comm
    T, N, _ = q.shape
    q_all = comm.all_gather(q.contiguous(), dim=1)  # heads of rank 0 first
    lens = local_context_len(md.positions, dcp, rank).to(torch.int32)
    bt = md.block_tables.index_select(0, md.req_id_per_token.long())
    qsl = torch.arange(T + 1, dtype=torch.int32, device=q.device)
    max_len = -(-md.max_seq_len // dcp)
    out, lse = ops.mla_attention(q_all, kv_cache, bt, lens, qsl, scale, kv_lora_rank, 1, max_len, lens, qsl,
                                 return_lse=True)
    lse_all = comm.all_gather(lse.float().unsqueeze(0).contiguous(), dim=0)  # [dcp, T, N * dcp]
    lse_g = torch.logsumexp(lse_all, 0)
    w = torch.exp(lse.float() - lse_g)
    w = torch.where(torch.isfinite(w), w, torch.zeros_like(w))
    part = (out.float() * w.unsqueeze(-1)).view(T, dcp, N, kv_lora_rank).transpose(0, 1).contiguous()
    mine = comm.reduce_scatter(part.view(dcp * T, N, kv_lora_rank), dim=0)  # sum over ranks of my head slice
    return mine.view(T, N, kv_lora_rank).to(q.dtype)
