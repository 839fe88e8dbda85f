"""DeepSeek-V2 / V3 / R1 / V3.2 (and GLM-MoE-DSA, Kimi-K2) : MLA attention + MoE with shared experts.

Reference: ``vllm_kunlun/models/deepseek_v2.py`` - MLP ``:100-146``, MoE with shared experts and
sigmoid group routing ``:149-308``, the sparse-attention indexer ``:475-788``, MLA wiring ``:791-960``,
weight loading (``fused_qkv_a_proj``, expert mapping, MTP layers skipped) ``:1285-1413`` - and the MLA
backends ``v1/attention/backends/mla/{common,flashmla,flashmla_sparse}.py``.

Decode, speculative verify and short prefill rows run in the weight-absorbed form over the latent cache
(``q_nope . W_UK`` -> 576-d MQA -> ``. W_UV``); requests with at least ``PREFILL_MIN_QUERY`` new tokens run in the
up-projected 192 / 128 form (``kv_b_proj`` applied to the keys, cached context read chunk by chunk through a bounded
workspace and merged by log-sum-exp).  The cache row is ``[kv_c (512) | k_pe (64)]``.  With ``index_topk > 0``
(V3.2) a lightning indexer selects the top-k context tokens per query and attention is restricted to them.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..ops.reference.basic import yarn_get_mscale
from ..parallel.state import get_state
from .dense import DenseDecoderLayer, GatedMLP
from .layers import (ColumnParallelLinear, RMSNorm, ReplicatedLinear, RowParallelLinear, get_cos_sin_cache, param)
from .moe import MoEForCausalLM, SparseMoEBlock


class Indexer(nn.Module):
    """Lightning indexer (``models/deepseek_v2.py:661-788``): 64 heads x 128 dims, LayerNorm on K, rotary
    on the first 64 dims, fp8 keys with a per-token scale in their own paged cache."""

    SP_MIN_TOKENS = 64   # tokens per rank from which the scoring is split over the tensor-parallel ranks

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.n_heads, self.head_dim, self.topk = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        self.rope_dim = cfg.qk_rope_head_dim
        self.wq_b = ReplicatedLinear(cfg.q_lora_rank, self.n_heads * self.head_dim, dtype=dtype, device=device)
        self.wk = ReplicatedLinear(cfg.hidden_size, self.head_dim, dtype=dtype, device=device)
        self.k_norm_weight = param(self.head_dim, dtype=dtype, device=device)
        self.k_norm_bias = param(self.head_dim, dtype=dtype, device=device)
        self.weights_proj = ReplicatedLinear(cfg.hidden_size, self.n_heads, dtype=dtype, device=device)
        self.softmax_scale = self.head_dim ** -0.5

    def forward(self, hidden, q_c, positions, cos_sin, k_cache, md):
        T = hidden.shape[0]
        k = self.wk(hidden)
        wscale = (self.n_heads ** -0.5) * self.softmax_scale
        if hidden.is_cuda and self.rope_dim == 64 and self.head_dim == 128:
            # one launch: K LayerNorm, rotary on q and k, e4m3 quantisation of both, key-cache write and the
            # per-(token, head) weight x scale product
            from ..ops import _ext
            from ..ops.mla_cuda import indexer_row_len, indexer_topk_cuda
            st = get_state()
            row_len = getattr(md, "_index_row_len", None)
            if row_len is None or row_len.shape[0] != T:   # the same for every layer of the step
                row_len = md._index_row_len = indexer_row_len(md.seq_lens, md.query_start_loc, md.req_id_per_token, T)
            max_len = min(int(md.max_seq_len), md.block_tables.shape[1] * k_cache.shape[1])
            tp = st.tp_size
            if tp > 1 and T >= self.SP_MIN_TOKENS * tp and not st.tp_comm.disabled:
                # prefill-sized batch: the indexer is replicated over the tensor-parallel ranks, so every rank
                # scores its slice of the tokens against the (complete, local) key cache and the selections are
                # all-gathered - 1 / tp of the scoring work and of the logits buffer per rank
                per = -(-T // tp)
                lo = min(T, st.tp_rank * per)
                hi = min(T, lo + per)
                ql = self.wq_b(q_c[lo:hi]).view(hi - lo, self.n_heads, self.head_dim)
                q_fp8, w = _ext.C().indexer_prep(ql, k, self.k_norm_weight, self.k_norm_bias, positions, cos_sin,
                                                 self.weights_proj(hidden[lo:hi]), wscale, k_cache, md.slot_mapping,
                                                 1e-6, True, lo)
                mine = torch.full((per, self.topk), -1, dtype=torch.int32, device=hidden.device)
                if hi > lo:
                    mine[: hi - lo] = indexer_topk_cuda(q_fp8, None, w, k_cache, md.block_tables, md.seq_lens,
                                                        md.query_start_loc, self.topk,
                                                        md.req_id_per_token[lo:hi].contiguous(), max_len,
                                                        row_len[lo:hi].contiguous(), lo, md.max_query_len)
                return st.tp_comm.all_gather(mine, dim=0)[:T].contiguous()
            q = self.wq_b(q_c).view(T, self.n_heads, self.head_dim)
            q_fp8, w = _ext.C().indexer_prep(q, k, self.k_norm_weight, self.k_norm_bias, positions, cos_sin,
                                             self.weights_proj(hidden), wscale, k_cache, md.slot_mapping, 1e-6, True, 0)
            return indexer_topk_cuda(q_fp8, None, w, k_cache, md.block_tables, md.seq_lens, md.query_start_loc,
                                     self.topk, md.req_id_per_token, max_len, row_len, 0, md.max_query_len)
        q = self.wq_b(q_c).view(T, self.n_heads, self.head_dim)
        k = torch.nn.functional.layer_norm(k.float(), (self.head_dim,), self.k_norm_weight.float(),
                                           self.k_norm_bias.float(), 1e-6).to(hidden.dtype)
        # rotary on the leading rope_dim dims of q and k (neox halves, as the reference indexer does)
        q_pe, k_pe = ops.rope(q[..., : self.rope_dim].reshape(T, -1).contiguous(),
                              k[:, : self.rope_dim].contiguous(), positions, cos_sin, self.rope_dim, True)
        q = torch.cat([q_pe.view(T, self.n_heads, self.rope_dim), q[..., self.rope_dim:]], -1)
        k = torch.cat([k_pe.view(T, self.rope_dim), k[:, self.rope_dim:]], -1)
        ops.indexer_k_quant_and_cache(k.contiguous(), k_cache, md.slot_mapping, True)
        q_fp8, q_scale = ops.quant_fp8_per_group(q.reshape(T * self.n_heads, self.head_dim).contiguous(), 128, True)
        weights = self.weights_proj(hidden).float() * wscale
        return ops.indexer_topk(q_fp8.view(T, self.n_heads, self.head_dim), q_scale.view(T, self.n_heads), weights,
                                k_cache, md.block_tables, md.seq_lens, md.query_start_loc, self.topk,
                                md.seq_lens_cpu, md.query_start_loc_cpu)


class MLAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        st = get_state()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.num_heads = cfg.num_heads // st.tp_size
        self.nope, self.rope, self.vdim, self.rank = (cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim,
                                                      cfg.kv_lora_rank)
        self.qk_dim = self.nope + self.rope
        H = cfg.hidden_size
        q = cfg.quantization
        if cfg.q_lora_rank:
            # checkpoint tensors q_a_proj + kv_a_proj_with_mqa are loaded into one replicated GEMM
            self.fused_qkv_a_proj = ReplicatedLinear(H, cfg.q_lora_rank + self.rank + self.rope, dtype=dtype,
                                                     device=device, quant=q)
            self.q_a_layernorm = RMSNorm(cfg.q_lora_rank, cfg.rms_norm_eps, dtype, device)
            self.q_b_proj = ColumnParallelLinear(cfg.q_lora_rank, [cfg.num_heads * self.qk_dim], dtype=dtype,
                                                 device=device, quant=q)
        else:
            self.q_proj = ColumnParallelLinear(H, [cfg.num_heads * self.qk_dim], dtype=dtype, device=device, quant=q)
            self.kv_a_proj_with_mqa = ReplicatedLinear(H, self.rank + self.rope, dtype=dtype, device=device, quant=q)
        self.kv_a_layernorm = RMSNorm(self.rank, cfg.rms_norm_eps, dtype, device)
        # kv_b_proj is kept in 16-bit and split into the absorbed factors after loading
        self.kv_b_proj = ColumnParallelLinear(self.rank, [cfg.num_heads * (self.nope + self.vdim)], dtype=dtype,
                                              device=device, quant=q)
        self.o_proj = RowParallelLinear(cfg.num_heads * self.vdim, H, dtype=dtype, device=device, quant=q,
                                        reduce_results=False)
        self.w_uk = self.w_uv = None  # [N, nope, rank] / [N, rank, vdim], built in finish()
        self.cos_sin = get_cos_sin_cache(self.rope, cfg.max_position, cfg.rope_theta, cfg.rope_scaling, device)
        scale = self.qk_dim ** -0.5
        rs = cfg.rope_scaling
        if rs.type == "yarn" and rs.mscale_all_dim:
            m = yarn_get_mscale(rs.factor, rs.mscale_all_dim)
            scale = scale * m * m
        self.scale = scale
        self.indexer = Indexer(cfg, dtype, device) if cfg.index_topk else None
        self._dtype = dtype

    def finish(self):
        """Absorb ``kv_b_proj`` (``mla/common.py:1423-1555``): ``W_UK [N, nope, rank]``, ``W_UV [N, rank, vdim]``."""
        m = self.kv_b_proj
        w = m.weight
        if w is None and getattr(m, "w4_packed", None) is not None:    # 4-bit checkpoint: the absorbed factors are 16-bit
            from ..quantization.int4 import dequant_w4
            w = dequant_w4(m.w4_packed.cpu(), m.w4_scale.cpu(), m.w4_zero.cpu(), m.w4_group).to(m.w4_packed.device)
        if w.dtype == torch.float8_e4m3fn:
            w = ops.reference_basic.dequant_fp8_block(w.cpu(), m.weight_scale_inv.cpu(), m.method.block).to(w.device)
        w = w.to(self._dtype).view(self.num_heads, self.nope + self.vdim, self.rank)
        self.w_uk = w[:, : self.nope].contiguous()                    # q_nope [T,N,nope] x [N,nope,rank]
        self.w_uv = w[:, self.nope:].transpose(1, 2).contiguous()     # out [T,N,rank] x [N,rank,vdim]
        # the up-projection itself, for the 192 / 128 prefill form (a view of the weight when that is 16-bit already)
        self.w_kvb = w.reshape(self.num_heads * (self.nope + self.vdim), self.rank)

    # ------------------------------------------------------------------ prefill in the up-projected form
    PREFILL_MIN_QUERY = 64            # requests with at least this many new tokens leave the absorbed form
    PREFILL_CTX_BYTES = 256 << 20     # bound of the up-projected context workspace (k_nope | v rows), bytes
    PREFILL_FORM = None               # None: on CUDA unless B200_MLA_PREFILL_FORM=0; True / False force it (tests)

    def _prefill_plan(self, md, kv_cache, on_cuda: bool):
        """Which requests of this step take the up-projected form, and the chunks their cached context is read in.
        Built once per step (every layer shares block tables and lengths) and kept in ``md.extras``.

        The absorbed form spends 576 + 512 multiply-adds per (query, key, head), the up-projected one 192 + 128 plus
        one ``kv_b_proj`` pass over the keys (``mla/common.py:1782-1843``); cached context (chunked prefill, prefix
        hits) is gathered from the paged latent cache chunk by chunk into a bounded workspace, up-projected,
        attended without a mask and merged by log-sum-exp (``mla/common.py:1614-1677``, workspace ``:467-495``)."""
        if "mla_prefill_plan" in md.extras:
            return md.extras["mla_prefill_plan"]
        plan = None
        if self.PREFILL_FORM is None:
            from .. import envs
            enabled = on_cuda and envs.B200_MLA_PREFILL_FORM
        else:
            enabled = self.PREFILL_FORM
        ok = (enabled and self.indexer is None and not md.is_dummy
              and ((self.nope, self.rope, self.vdim) == (128, 64, 128) or not on_cuda)   # the kernel's shape and md.max_query_len >= self.PREFILL_MIN_QUERY
              and md.seq_lens_cpu is not None and md.query_start_loc_cpu is not None
              and not (kv_cache.dtype == torch.uint8 and not on_cuda))
        if ok:
            import numpy as np
            dev = kv_cache.device
            B = md.num_reqs
            qsl = md.query_start_loc_cpu.numpy().astype(np.int64)[: B + 1]
            sl = md.seq_lens_cpu.numpy().astype(np.int64)[:B]
            ql = qsl[1:] - qsl[:-1]
            pre = np.nonzero(ql >= self.PREFILL_MIN_QUERY)[0]
            rest = np.nonzero((ql < self.PREFILL_MIN_QUERY) & (ql > 0))[0]

            def dev_i32(a):
                return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)

            def dev_i64(a):
                return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int64)).to(dev)

            plan = {"all": len(rest) == 0 and len(pre) == B}
            qlp = ql[pre]
            qsl_p = np.concatenate([[0], np.cumsum(qlp)])
            plan["tok"] = None if plan["all"] else dev_i64(np.concatenate([np.arange(qsl[r], qsl[r + 1]) for r in pre]))
            plan["qsl"] = dev_i32(qsl_p)
            plan["kv_starts"] = dev_i32(qsl_p[:-1])
            plan["kv_lens"] = dev_i32(qlp)
            plan["qsl_cpu"], plan["q_lens_cpu"] = qsl_p, qlp
            plan["max_q"] = int(qlp.max())
            # cached context of the prefill requests, in chunks that fit the workspace
            ctx = (sl - ql)[pre]
            chunks = []
            n_ctx = int((ctx > 0).sum())
            if n_ctx:
                bs = kv_cache.shape[1]
                budget = max(64, self.PREFILL_CTX_BYTES // (self.num_heads * (self.nope + self.vdim) * 2))
                per_req = max(64, budget // n_ctx // 64 * 64)
                for lo in range(0, int(ctx.max()), per_req):
                    a = np.minimum(ctx, lo)
                    b = np.minimum(ctx, lo + per_req)
                    lens = b - a
                    req = np.repeat(pre, lens)
                    pos = np.concatenate([np.arange(x, y) for x, y in zip(a, b)])
                    req_d, pos_d = dev_i64(req), dev_i64(pos)
                    slots = (md.block_tables[req_d, pos_d // bs].long() * bs + pos_d % bs).to(torch.int32)
                    starts = np.concatenate([[0], np.cumsum(lens)])[:-1]
                    chunks.append({"slots": slots, "kv_starts": dev_i32(starts), "kv_lens": dev_i32(lens),
                                   "starts_cpu": starts, "lens_cpu": lens})
            plan["chunks"] = chunks
            # the other requests of a mixed step keep the absorbed form over a compacted sub-batch
            if len(rest):
                qlr = ql[rest]
                qsl_r = np.concatenate([[0], np.cumsum(qlr)])
                rest_d = dev_i64(rest)
                plan["rest"] = {
                    "tok": dev_i64(np.concatenate([np.arange(qsl[r], qsl[r + 1]) for r in rest])),
                    "block_tables": md.block_tables.index_select(0, rest_d).contiguous(),
                    "seq_lens": dev_i32(sl[rest]), "qsl": dev_i32(qsl_r),
                    "seq_lens_cpu": torch.from_numpy(sl[rest].astype(np.int32)),
                    "qsl_cpu": torch.from_numpy(qsl_r.astype(np.int32)),
                    "max_q": int(qlr.max()), "max_seq": int(sl[rest].max())}
            else:
                plan["rest"] = None
        md.extras["mla_prefill_plan"] = plan
        return plan

    def _attend_prefill(self, plan, q_nope, q_pe, kv_c, k_pe, kv_cache):
        """Attention of the plan's prefill requests in the up-projected form -> ``[Tp, N, vdim]``."""
        N = self.num_heads
        tok = plan["tok"]
        if tok is not None:
            q_nope, q_pe, kv_c, k_pe = (x.index_select(0, tok) for x in (q_nope, q_pe, kv_c, k_pe))
        Tp = q_nope.shape[0]
        q = torch.cat([q_nope, q_pe.view(Tp, N, self.rope)], -1)
        cpu = not q.is_cuda
        # the new tokens among themselves (causal)
        kv_new = ops.linear(kv_c.contiguous(), self.w_kvb)
        out, lse = ops.mla_prefill_attention(q, kv_new, k_pe.contiguous(),
                                             plan["qsl_cpu"][:-1] if cpu else plan["kv_starts"],
                                             plan["q_lens_cpu"] if cpu else plan["kv_lens"],
                                             plan["qsl_cpu"] if cpu else plan["qsl"], True, self.scale, plan["max_q"])
        del kv_new
        # cached context, chunk by chunk through the bounded workspace (no mask), merged by log-sum-exp
        for ch in plan["chunks"]:
            n = ch["slots"].shape[0]
            if cpu:
                rows = kv_cache.reshape(-1, kv_cache.shape[-1])[ch["slots"].long()]
            else:
                from ..ops import _ext
                rows = torch.empty(n, self.rank + self.rope, dtype=q.dtype, device=q.device)
                _ext.C().gather_mla_rows(rows, kv_cache, ch["slots"])
            kv_ctx = ops.linear(rows[:, : self.rank].contiguous(), self.w_kvb)
            o_c, lse_c = ops.mla_prefill_attention(q, kv_ctx, rows[:, self.rank:],
                                                   ch["starts_cpu"] if cpu else ch["kv_starts"],
                                                   ch["lens_cpu"] if cpu else ch["kv_lens"],
                                                   plan["qsl_cpu"] if cpu else plan["qsl"], False, self.scale,
                                                   plan["max_q"])
            out, lse = ops.merge_attn_states(out, lse, o_c, lse_c)
        return out

    FP8_GATHER_TOKENS = 256   # query tokens per pass of the fp8-cache path (scratch: tokens x top-k x 1152 bytes)

    def _sparse_fp8(self, qf, kv_cache, slots):
        """Sparse attention over the `fp8_ds_mla` cache: the selected rows of a group of query tokens are gathered
        and de-quantised into a dense 16-bit scratch (one kernel), and the sparse kernel then runs over the scratch
        with positional indices.  The scratch is bounded by ``FP8_GATHER_TOKENS``; long prefill chunks take several
        passes."""
        T, topk = slots.shape
        out = torch.empty(T, self.num_heads, self.rank, dtype=qf.dtype, device=qf.device)
        step = min(T, self.FP8_GATHER_TOKENS)
        if qf.is_cuda:
            from ..ops import _ext
            scratch = torch.empty(step * topk, 576, dtype=qf.dtype, device=qf.device)
            pos = torch.arange(step * topk, dtype=torch.int32, device=qf.device).view(step, topk)
        for t0 in range(0, T, step):
            t1 = min(T, t0 + step)
            sl = slots[t0:t1].contiguous()
            if qf.is_cuda:
                rows = scratch[: (t1 - t0) * topk]
                _ext.C().gather_mla_rows(rows, kv_cache, sl.view(-1))
                idx = torch.where(sl >= 0, pos[: t1 - t0], torch.full_like(sl, -1))
                out[t0:t1] = ops.sparse_mla_attention(qf[t0:t1].contiguous(), rows, idx, self.scale, self.rank)
            else:
                out[t0:t1] = ops.sparse_mla_attention(qf[t0:t1], kv_cache, sl, self.scale, self.rank)
        return out

    def forward(self, hidden):
        ctx = get_forward_context()
        md = ctx.attn
        cache = ctx.kv_caches[self.layer_idx]
        kv_cache, idx_cache = (cache if isinstance(cache, tuple) else (cache, None))
        T = hidden.shape[0]
        cfg = self.cfg
        if cfg.q_lora_rank:
            qkv_a = self.fused_qkv_a_proj(hidden)
            q_c = self.q_a_layernorm(qkv_a[:, : cfg.q_lora_rank].contiguous())
            kv_c, k_pe = qkv_a[:, cfg.q_lora_rank: cfg.q_lora_rank + self.rank], qkv_a[:, cfg.q_lora_rank + self.rank:]
            q = self.q_b_proj(q_c)
        else:
            q_c = None
            q = self.q_proj(hidden)
            kv = self.kv_a_proj_with_mqa(hidden)
            kv_c, k_pe = kv[:, : self.rank], kv[:, self.rank:]
        kv_c = self.kv_a_layernorm(kv_c.contiguous())
        q = q.view(T, self.num_heads, self.qk_dim)
        q_nope, q_pe = q[..., : self.nope], q[..., self.nope:]
        q_pe, k_pe = ops.rope(q_pe.reshape(T, -1).contiguous(), k_pe.contiguous(), md.positions, self.cos_sin,
                              self.rope, cfg.rope_neox)
        ops.concat_and_cache_mla(kv_c, k_pe, kv_cache, md.slot_mapping)
        plan = None
        if self.indexer is None and ctx.pstate.dcp_size == 1 and md.max_query_len >= self.PREFILL_MIN_QUERY:
            plan = self._prefill_plan(md, kv_cache, hidden.is_cuda)
        if plan is not None:
            o_p = self._attend_prefill(plan, q_nope, q_pe, kv_c, k_pe, kv_cache)
            rest = plan["rest"]
            if plan["all"]:
                v = o_p
            else:
                v = torch.zeros(T, self.num_heads, self.vdim, dtype=o_p.dtype, device=o_p.device)
                v.index_copy_(0, plan["tok"], o_p)
                if rest is not None:   # decode / short rows of a mixed step: the absorbed form over a sub-batch
                    qn = q_nope.index_select(0, rest["tok"])
                    qp = q_pe.view(T, self.num_heads, self.rope).index_select(0, rest["tok"])
                    qf = torch.cat([ops.bmm_heads(qn, self.w_uk), qp], -1).contiguous()
                    o = ops.mla_attention(qf, kv_cache, rest["block_tables"], rest["seq_lens"], rest["qsl"], self.scale,
                                          self.rank, rest["max_q"], rest["max_seq"], rest["seq_lens_cpu"],
                                          rest["qsl_cpu"], md.workspace)
                    v.index_copy_(0, rest["tok"], ops.bmm_heads(o, self.w_uv))
            return self.o_proj(v.reshape(T, self.num_heads * self.vdim))
        # absorbed query: [T, N, rank] = q_nope . W_UK   (batched over heads)
        ql = ops.bmm_heads(q_nope, self.w_uk)
        qf = torch.cat([ql, q_pe.view(T, self.num_heads, self.rope)], -1)
        if self.indexer is not None:
            local_idx = self.indexer(hidden, q_c, md.positions, self.cos_sin, idx_cache, md)
            slots = ops.convert_req_index_to_global_index(md.req_id_per_token, md.block_tables, local_idx,
                                                          kv_cache.shape[1])
            if kv_cache.dtype == torch.uint8:
                o = self._sparse_fp8(qf.contiguous(), kv_cache, slots)
            else:
                o = ops.sparse_mla_attention(qf.contiguous(), kv_cache, slots, self.scale, self.rank)
        elif ctx.pstate.dcp_size > 1:
            from ..attention.dcp import dcp_mla_attention
            o = dcp_mla_attention(qf.contiguous(), kv_cache, md, self.scale, self.rank, ctx.pstate)
        else:
            o = ops.mla_attention(qf.contiguous(), kv_cache, md.block_tables, md.seq_lens, md.query_start_loc,
                                  self.scale, self.rank, md.max_query_len, md.max_seq_len, md.seq_lens_cpu,
                                  md.query_start_loc_cpu, md.workspace, stable_metadata=True)
        v = ops.bmm_heads(o, self.w_uv)  # [T, N, vdim]
        return self.o_proj(v.reshape(T, self.num_heads * self.vdim))


class DeepseekDecoderLayer(DenseDecoderLayer):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        nn.Module.__init__(self)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = MLAAttention(cfg, layer_idx, dtype, device) if cfg.use_mla else None
        if self.self_attn is None:
            from .dense import GQAAttention
            self.self_attn = GQAAttention(cfg, layer_idx, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.mlp = self.build_mlp(cfg, layer_idx, dtype, device)

    def build_mlp(self, cfg, layer_idx, dtype, device):
        if cfg.layer_is_moe(layer_idx):
            return SparseMoEBlock(cfg, dtype, device)
        return GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quantization, "silu",
                        reduce_results=False)


class DeepseekForCausalLM(MoEForCausalLM):
    layer_cls = DeepseekDecoderLayer

    def kv_cache_spec(self, block_size: int):
        cfg = self.cfg
        if not cfg.use_mla:
            return super().kv_cache_spec(block_size)
        spec = {}
        # `fp8_ds_mla` (sparse-attention models only): 656-byte rows = 4 x 128 e4m3 | 4 f32 scales | 64 bf16 rope dims
        fp8 = getattr(self, "kv_cache_dtype", "auto") == "fp8_ds_mla"
        if fp8 and not cfg.index_topk:
            raise ValueError("kv_cache_dtype='fp8_ds_mla' is served for sparse-attention (indexer) models only")
        for i in range(self.first_layer, self.last_layer):
            main = ((block_size, 656), torch.uint8) if fp8 else ((block_size, cfg.mla_cache_dim), self.dtype)
            spec[i] = [main, ((block_size, 132), torch.uint8)] if cfg.index_topk else main
        return spec

    def finish_loading(self):
        super().finish_loading()
        for m in self.modules():
            if isinstance(m, MLAAttention):
                m.finish()

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        """Checkpoint specifics (``models/deepseek_v2.py:1285-1413``): ``q_a_proj`` and
        ``kv_a_proj_with_mqa`` stack into ``fused_qkv_a_proj``; layers past ``num_layers`` (MTP) are skipped;
        ``mlp.gate.weight`` is the router."""
        cfg = self.cfg
        pending = {}
        out = []
        for name, w in weights:
            parts = name.split(".")
            if len(parts) > 2 and parts[1] == "layers" and parts[2].isdigit() and int(parts[2]) >= cfg.num_layers:
                continue  # multi-token-prediction layers live in DeepSeekMTP
            if cfg.q_lora_rank and (".q_a_proj." in name or ".kv_a_proj_with_mqa." in name):
                key = name.replace(".q_a_proj.", ".fused_qkv_a_proj.").replace(".kv_a_proj_with_mqa.",
                                                                               ".fused_qkv_a_proj.")
                slot = 0 if ".q_a_proj." in name else 1
                pending.setdefault(key, {})[slot] = w
                if len(pending[key]) == 2:
                    out.append((key, torch.cat([pending[key][0], pending[key][1]], 0)))
                    del pending[key]
                continue
            name = name.replace(".indexer.k_norm.weight", ".indexer.k_norm_weight")
            name = name.replace(".indexer.k_norm.bias", ".indexer.k_norm_bias")
            out.append((name, w))
        return super().load_weights(out)
