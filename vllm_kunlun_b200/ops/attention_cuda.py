"""CUDA paged attention entry (``csrc/attention/paged_attention.cu``).

Batches are decode-first; a decode-only batch uses the decode warp layout with split-KV sized to
fill the SMs, a prefill batch uses the 64-row layout.  Split-KV partials live in a workspace that
the caller may pre-allocate (needed under CUDA-graph capture).
"""
from __future__ import annotations

from typing import Optional

import torch

import os

from . import _ext

_SM_COUNT: dict = {}
# decode-shaped calls with head dim 128 and cache blocks of a multiple of 64 tokens run on the tcgen05 kernel
# (csrc/attention/decode_umma.cu); B200_ATTN_UMMA=0 keeps them on the mma.sync kernel
UMMA_DECODE = [os.environ.get("B200_ATTN_UMMA", "1") != "0"]
# prefill-shaped calls (same head dim / block constraints) run on csrc/attention/prefill_umma.cu;
# B200_PREFILL_UMMA=0 keeps them on the mma.sync kernel
UMMA_PREFILL = [os.environ.get("B200_PREFILL_UMMA", "1") != "0"]


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


class AttnWorkspace:
    """Split-KV scratch: ``ws_o [splits, T, Hq, D]`` fp32 and ``ws_lse [splits, T, Hq]``."""

    def __init__(self, max_tokens: int, num_heads: int, head_dim: int, max_splits: int, device):
        self.max_splits = max_splits
        self.max_tokens = max_tokens
        self.o = torch.empty(max_splits * max_tokens * num_heads * head_dim, dtype=torch.float32, device=device)
        self.lse = torch.empty(max_splits * max_tokens * num_heads, dtype=torch.float32, device=device)


def plan_splits(num_reqs: int, num_kv_heads: int, q_tiles: int, max_seq_len: int, device, max_splits: int = 16,
                ctas_per_sm: int = 2, warps: int = 4, tile: int = 16) -> int:
    """Split count for decode: fill the resident CTA slots in whole waves while every warp keeps
    enough 16-key tiles to amortise its pipeline prologue."""
    base = max(1, num_reqs * num_kv_heads * q_tiles)
    slots = sm_count(device) * ctas_per_sm
    best, best_score = 1, -1.0
    for s in range(1, max_splits + 1):
        ctas = base * s
        waves = -(-ctas // slots)
        eff = ctas / (waves * slots)
        tiles_per_warp = max_seq_len / tile / warps / s
        score = eff * tiles_per_warp / (tiles_per_warp + 3.0)
        if score > best_score + 1e-9:
            best, best_score = s, score
    return best


def plan_splits_umma(num_reqs: int, num_kv_heads: int, max_seq_len: int, device, max_splits: int = 16) -> int:
    """One CTA per SM streams 128-key tiles through a deep TMA ring, so a (request, kv head) pair is split only as
    far as it takes to occupy the SMs, and never below two tiles per CTA."""
    base = max(1, num_reqs * num_kv_heads)
    tiles = max(1, -(-max_seq_len // 128))
    s = max(1, sm_count(device) // base)
    return int(max(1, min(s, max_splits, max(1, tiles // 2))))


def paged_attention_cuda(out, q, kv_cache, block_tables, seq_lens, query_start_loc, scale: float,
                         max_query_len: int, max_seq_len: int, window: Optional[int] = None, sinks=None,
                         workspace: Optional[AttnWorkspace] = None, num_splits: Optional[int] = None,
                         stable_metadata: bool = False):
    """``stable_metadata``: the caller promises that ``block_tables`` / ``seq_lens`` / ``query_start_loc`` were
    filled by host copies before the step's first kernel (as the engine's runner does) and that the cache rows of
    the old context come from earlier steps; the decode kernel then starts fetching KV tiles while the kernel in
    front of it is still running."""
    T, Hq, D = q.shape
    Hkv = kv_cache.shape[2]
    g = Hq // Hkv
    B = seq_lens.shape[0]
    decode_layout = max_query_len * g <= 16
    if (decode_layout and UMMA_DECODE[0] and D == 128 and kv_cache.shape[3] % 64 == 0
            and q.dtype in (torch.bfloat16, torch.float16)):
        if num_splits is None:
            num_splits = plan_splits_umma(B, Hkv, max_seq_len, q.device,
                                          workspace.max_splits if workspace is not None else 16)
        ws_o = ws_lse = None
        if num_splits > 1:
            if workspace is None or T > workspace.max_tokens or num_splits > workspace.max_splits:
                # e.g. several requests whose last prefill chunk is only a few tokens long: more rows in decode
                # layout than the step's decode batch was sized for
                workspace = AttnWorkspace(T, Hq, D, num_splits, q.device)
            ws_o, ws_lse = workspace.o, workspace.lse
        _ext.C().decode_attention_umma(out, q, kv_cache, block_tables, seq_lens, query_start_loc, sinks, ws_o, ws_lse,
                                       max_query_len, num_splits, window or 0, scale, bool(stable_metadata))
        return out
    if (not decode_layout and UMMA_PREFILL[0] and D == 128 and kv_cache.shape[3] % 64 == 0 and kv_cache.dim() == 5
            and q.dtype in (torch.bfloat16, torch.float16) and q.is_contiguous() and out.is_contiguous()
            and kv_cache.is_contiguous()):
        # prefill / chunked prefill on tcgen05: 128 query rows of one head per CTA, S and O in TMEM
        _ext.C().prefill_attention_umma(out, q, kv_cache, block_tables, seq_lens, query_start_loc, sinks, None,
                                        max_query_len, window or 0, scale)
        return out
    if num_splits is None:
        if decode_layout:
            num_splits = plan_splits(B, Hkv, 1, max_seq_len, q.device,
                                     workspace.max_splits if workspace is not None else 16)
        else:
            num_splits = 1
    ws_o = ws_lse = None
    if num_splits > 1:
        if workspace is None or T > workspace.max_tokens or num_splits > workspace.max_splits:
            # e.g. several requests whose last prefill chunk is only a few tokens long: more rows in decode
            # layout than the step's decode batch was sized for
            workspace = AttnWorkspace(T, Hq, D, num_splits, q.device)
        ws_o, ws_lse = workspace.o, workspace.lse
    _ext.C().paged_attention(out, q, kv_cache, block_tables, seq_lens, query_start_loc, sinks, ws_o, ws_lse,
                             max_query_len, num_splits, window or 0, scale, decode_layout)
    return out
