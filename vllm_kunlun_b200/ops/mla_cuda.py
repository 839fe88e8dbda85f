"""CUDA entries of the MLA family: absorbed attention over the latent cache (dense paged and sparse),
the per-head absorption products and the lightning-indexer scoring.

Kernels: ``csrc/attention/mla_attention.cu`` (one kernel for dense and sparse key sources, split-KV)
and the grouped tcgen05 GEMM (``csrc/gemm/gemm_grouped.cu``) with heads as groups for
``q_nope . W_UK`` / ``o . W_UV``."""
from __future__ import annotations

import torch

from . import _ext
from .attention_cuda import sm_count

_LOD: dict = {}


def _splits(ctas: int, tiles: int, device, cap: int = 16) -> int:
    want = -(-2 * sm_count(device) // max(1, ctas))
    return int(max(1, min(want, cap, max(1, tiles // 2))))


def _ws(T, N, splits, device):
    return (torch.empty(splits * T * N * 512, dtype=torch.float32, device=device),
            torch.empty(splits * T * N, dtype=torch.float32, device=device))


# decode / speculative-verify batches over 64-token cache blocks run on the tcgen05 kernel
# (csrc/attention/mla_decode_umma.cu); B200_MLA_UMMA=0 keeps them on the mma.sync kernel
import os as _os
UMMA_DECODE = [_os.environ.get("B200_MLA_UMMA", "1") != "0"]
_UMMA_MAX_QLEN = 4
_FORCE_WORKSPACE = [False]  # tests: merge 2/4/8 splits through the global workspace instead of the cluster


_MAX_CLUSTERS: dict = {}


def _max_clusters(R: int, S: int, dtype, device) -> int:
    key = (R, S, dtype, str(device))
    n = _MAX_CLUSTERS.get(key)
    if n is None:
        with torch.cuda.device(device):
            n = _MAX_CLUSTERS[key] = int(_ext.C().mla_decode_max_clusters(R, S, 2 if dtype == torch.float16 else 1))
    return n


def plan_mla_splits(units: int, tiles: int, R: int, dtype, device):
    """``(num_splits, merge in a cluster?)`` for ``units`` (request, head group) pairs of ``tiles`` cache pages.

    Splits of one unit either form a thread-block cluster of 2 / 4 / 8 CTAs that merges in shared memory - only
    when every cluster of the launch is resident at once (the device holds fewer clusters of 8 than SMs / 8:
    a cluster lives inside one GPC) - or go through a workspace that the last CTA to finish combines, which costs
    about three more pages of time.  The cheaper of the two estimates wins."""
    sms = sm_count(device)
    cap = max(1, tiles // 2)
    best = (1, False, tiles)
    for S in (2, 4, 8):
        if S <= cap and units <= _max_clusters(R, S, dtype, device):
            cost = -(-tiles // S)
            if cost < best[2]:
                best = (S, True, cost)
    Sw = int(max(1, min(sms // max(1, units), 16, cap)))
    if Sw > 1:
        cost = -(-tiles // Sw) + 3
        if cost < best[2]:
            best = (Sw, False, cost)
    return best[0], best[1]


def mla_decode_umma(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, max_query_len, max_seq_len,
                    num_splits=None, stable_metadata: bool = False):
    """Dense paged MLA decode on tcgen05: every request has at most ``max_query_len`` (<= 4) query tokens."""
    T, N, _ = q.shape
    B = seq_lens.shape[0]
    out = torch.empty(T, N, 512, dtype=q.dtype, device=q.device)
    R = 16 if N * max_query_len <= 16 else 32
    groups = -(-N // (R // max_query_len))
    if num_splits is None:
        num_splits, cluster = plan_mla_splits(groups * B, max(1, -(-max_seq_len // 64)), R, q.dtype, q.device)
    else:
        cluster = num_splits in (2, 4, 8) and groups * B <= _max_clusters(R, num_splits, q.dtype, q.device)
    cluster = cluster and not _FORCE_WORKSPACE[0]
    ws_o, ws_lse = _ws(T, N, num_splits, q.device) if num_splits > 1 and not cluster else (None, None)
    _ext.C().mla_decode_umma(out, q, kv_cache, block_tables, seq_lens, query_start_loc, ws_o, ws_lse, max_query_len,
                             num_splits, scale, bool(stable_metadata))
    return out


def mla_attention_cuda(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, kv_lora_rank, max_query_len,
                       max_seq_len, workspace=None, req_of_token=None, return_lse: bool = False,
                       stable_metadata: bool = False):
    assert kv_lora_rank == 512 and q.shape[-1] == 576 and kv_cache.dtype == q.dtype
    T, N, _ = q.shape
    if (UMMA_DECODE[0] and not return_lse and 1 <= max_query_len <= _UMMA_MAX_QLEN and kv_cache.dim() == 3
            and kv_cache.shape[1] == 64 and q.is_contiguous() and kv_cache.is_contiguous()):
        return mla_decode_umma(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, max_query_len, max_seq_len,
                               stable_metadata=stable_metadata)
    if req_of_token is None:
        lens = (query_start_loc[1:] - query_start_loc[:-1]).long()
        req_of_token = torch.repeat_interleave(torch.arange(lens.shape[0], device=q.device, dtype=torch.int32), lens,
                                               output_size=T)
    out = torch.empty(T, N, 512, dtype=q.dtype, device=q.device)
    splits = _splits(-(-N // 16) * T, -(-max_seq_len // 32), q.device)
    if return_lse:
        splits = max(splits, 2)  # the split-KV path keeps per-split log-sum-exps (base 2) in the workspace
    ws_o, ws_lse = _ws(T, N, splits, q.device) if splits > 1 else (None, None)
    _ext.C().mla_attention(out, q, kv_cache, block_tables, seq_lens, query_start_loc, req_of_token, None, ws_o, ws_lse,
                           splits, scale)
    if not return_lse:
        return out
    lse = torch.logsumexp(ws_lse.view(splits, T, N) * 0.6931471805599453, 0)
    empty = torch.isinf(lse) & (lse < 0)
    return torch.where(empty.unsqueeze(-1), torch.zeros_like(out), out), lse


def sparse_mla_cuda(q, kv_flat, indices, scale, d_v=512):
    assert d_v == 512 and kv_flat.dtype == q.dtype, "sparse MLA kernel reads the 16-bit latent cache"
    T, N, _ = q.shape
    out = torch.empty(T, N, 512, dtype=q.dtype, device=q.device)
    topk = indices.shape[1]
    splits = _splits(-(-N // 16) * T, -(-topk // 32), q.device)
    ws_o, ws_lse = _ws(T, N, splits, q.device) if splits > 1 else (None, None)
    _ext.C().mla_attention(out, q, kv_flat, None, None, None, None, indices.contiguous(), ws_o, ws_lse, splits, scale)
    return out


def bmm_heads_cuda(x, w):
    """``out[t, n, :] = x[t, n, :] @ w[n]`` with ``w [N, K, D]``: heads are the groups of a grouped GEMM."""
    T, N, K = x.shape
    D = w.shape[2]
    # K-major copy [N, D, K], made once per weight and kept ON the weight tensor: a cache keyed by address would hand
    # a later model the copy of an earlier one whose (freed) weight lived at the same address
    wt = getattr(w, "_b200_kmajor", None)
    if wt is None or wt.shape != (N, D, K):
        wt = w.transpose(1, 2).contiguous()
        w._b200_kmajor = wt
    lk = (N, T, str(x.device))
    lod = _LOD.get(lk)
    if lod is None:
        lod = (torch.arange(N + 1, dtype=torch.int32, device=x.device) * T).contiguous()
        _LOD[lk] = lod
    xs = x.transpose(0, 1).contiguous().view(N * T, K)
    out = torch.empty(N * T, D, dtype=x.dtype, device=x.device)
    _ext.C().grouped_gemm(out, xs, wt, lod, None, None, None, 0)
    return out.view(N, T, D).transpose(0, 1)


def indexer_row_len(seq_lens, query_start_loc, req_of_token, T):
    """Keys visible to token ``t``: its position + 1 (int32 ``[T]``); the same for every layer of a step."""
    rt = req_of_token.long()
    qs = query_start_loc.long()[rt]
    q_len = (query_start_loc[1:] - query_start_loc[:-1]).long()[rt]
    return (seq_lens.long()[rt] - q_len + (torch.arange(T, device=seq_lens.device) - qs) + 1).to(torch.int32).contiguous()


# prefill-sized batches score on the tcgen05 kernel (csrc/attention/indexer_umma.cu); B200_INDEXER_UMMA=0 keeps
# everything on the mma.sync kernel
INDEXER_UMMA = [_os.environ.get("B200_INDEXER_UMMA", "1") != "0"]
_INDEXER_UMMA_MIN_ROWS = 64


def indexer_topk_cuda(q_fp8, q_scale, weights, k_cache, block_tables, seq_lens, query_start_loc, topk,
                      req_of_token=None, max_len=None, row_len=None, t0: int = 0, max_query_len=None):
    """fp8 scoring (``csrc/attention/indexer.cu``) + radix-select top-k; request-local indices ``[T, topk]``.
    ``q_scale=None``: ``weights`` already holds ``head weight x q scale`` (``indexer_prep``).  ``t0``: the rows are
    tokens ``t0 .. t0 + T`` of the batch (``req_of_token`` / ``row_len`` are the matching slices)."""
    T, H, D = q_fp8.shape
    assert H == 64 and D == 128, "indexer kernel is specialised for 64 heads x 128 dims"
    if req_of_token is None:
        lens = (query_start_loc[1:] - query_start_loc[:-1]).long()
        req_of_token = torch.repeat_interleave(torch.arange(lens.shape[0], device=q_fp8.device, dtype=torch.int32),
                                               lens, output_size=T)
    if max_len is None:
        max_len = block_tables.shape[1] * k_cache.shape[1]
    ld = -(-max_len // 512) * 512
    logits = torch.empty(T, ld, dtype=torch.float32, device=q_fp8.device)
    w = weights if q_scale is None else (weights.float() * q_scale.float()).contiguous()
    C = _ext.C()
    if row_len is None:
        assert t0 == 0
        row_len = indexer_row_len(seq_lens, query_start_loc, req_of_token, T)
    if (INDEXER_UMMA[0] and max_query_len is not None and T >= _INDEXER_UMMA_MIN_ROWS and k_cache.shape[1] == 64
            and w.is_contiguous()):
        # keys on the UMMA M side, 4 tokens x 64 heads on the N side; writes keys [0, n_keys) of every row only,
        # which is all that the selection below reads
        C.indexer_logits_umma(logits, q_fp8.view(torch.uint8).contiguous(), w, k_cache, block_tables, seq_lens,
                              query_start_loc, int(max_query_len), t0)
    else:
        C.indexer_logits(logits, q_fp8.view(torch.uint8).contiguous(), w, k_cache, block_tables, seq_lens,
                         query_start_loc, req_of_token, t0)
    out = torch.empty(T, topk, dtype=torch.int32, device=q_fp8.device)
    C.topk_rows(out, logits, row_len)
    return out
