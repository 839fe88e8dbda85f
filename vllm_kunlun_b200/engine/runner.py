"""Model runner: owns the model shard, the KV cache, per-step input staging and CUDA graphs.

Counterpart of upstream's ``GPUModelRunner`` that the reference plugs into (call stack in
``v1/attention/backends/kunlun_attn.py:587-670``: per-step host metadata with several small H2D
copies).  Here all integer metadata of a step is packed into two pinned staging buffers and moved
with two async copies into persistent device buffers, so that the same tensors can be bound into a
captured decode graph.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..attention.metadata import AttentionMetadata, ForwardContext, set_forward_context
from ..config import EngineConfig, cdiv, round_up
from ..models import build_model
from ..parallel.state import ParallelState, get_state
from ..sample.sampler import Sampler
from .scheduler import SchedulerOutput


@dataclass
class StepHandle:
    """Result of one launched step.  ``tokens`` stays on the device; ``tokens_cpu`` is filled by an
    async copy guarded by ``event`` (CUDA) or immediately (CPU)."""

    sched: SchedulerOutput
    sample_reqs: list  # requests in the row order of ``tokens``
    rows_per_req: list  # number of sampled rows per request (1, or 1 + drafts)
    tokens: torch.Tensor
    tokens_cpu: torch.Tensor
    event: Optional[object]
    hidden: Optional[torch.Tensor] = None  # last hidden states of sampled rows
    launch_time: float = 0.0
    md: Optional[object] = None            # kept for the draft model (speculative decoding)
    input_ids: Optional[torch.Tensor] = None
    full_hidden: Optional[torch.Tensor] = None
    logprobs_cpu: Optional[torch.Tensor] = None  # log p of every sampled row (when a request asked for it)
    status_cpu: Optional[torch.Tensor] = None    # device status words copied with the tokens (0 = all waits were met)
    status_names: tuple = ()

    def wait(self) -> torch.Tensor:
        if self.event is not None:
            self.event.synchronize()
        if self.status_cpu is not None:
            codes = self.status_cpu.tolist()
            if any(codes):
                bad = ", ".join(f"{n}={c}" for n, c in zip(self.status_names, codes) if c)
                raise DeviceWaitTimeout(f"a bounded device-side wait timed out during this step ({bad}); "
                                        "the tokens of the step are not trustworthy")
        return self.tokens_cpu


class DeviceWaitTimeout(RuntimeError):
    """A kernel gave up on a bounded wait (peer flag, mbarrier) and finished with wrong data."""


class ModelRunner:
    def __init__(self, cfg: EngineConfig, pstate: Optional[ParallelState] = None):
        self.cfg = cfg
        self.pstate = pstate or get_state()
        self.device = torch.device(cfg.device)
        self.is_cuda = self.device.type == "cuda"
        m = cfg.model
        with torch.inference_mode():
            self.model = build_model(m, device=cfg.device)
            if cfg.weights_path:
                from ..models.loader import load_safetensors
                self.model.load_weights(load_safetensors(cfg.weights_path))
            else:
                self.model.init_random(cfg.seed, cfg.init_std)
        self.model.kv_cache_dtype = cfg.cache.cache_dtype   # read by kv_cache_spec (e.g. "fp8_ds_mla")
        self.block_size = cfg.cache.block_size
        self.dcp, self.dcp_rank = self.pstate.dcp_size, self.pstate.dcp_rank
        if self.dcp > 1:
            assert m.use_mla and not m.index_topk, "decode context parallelism serves dense MLA models"
        self.tokens_per_block = self.block_size * self.dcp
        self.max_bs = cfg.scheduler.max_num_seqs
        self.max_tokens = cfg.scheduler.max_num_batched_tokens
        self.num_spec = cfg.speculative.num_speculative_tokens
        # a verify step may run num_spec draft positions past the last allowed token
        self.max_blocks_per_seq = cdiv(cfg.scheduler.max_model_len + self.num_spec, self.tokens_per_block)
        self.sampler = Sampler(m.vocab_size, self.device, seed=cfg.seed)
        self.num_blocks = self._plan_num_blocks()
        self.kv_caches = self._alloc_kv()
        self.num_state_slots = 0
        if getattr(self.model, "uses_state_cache", False):
            # one slot per running request for the linear-attention (conv + recurrent) state
            self.num_state_slots = self.max_bs
            for i, specs in self.model.state_cache_spec().items():
                self.kv_caches[i] = tuple(torch.zeros((self.num_state_slots, *shp), dtype=dt, device=self.device)
                                          for shp, dt in specs)
        self._alloc_staging()
        self.graphs = None
        self.is_vl = hasattr(self.model, "embed_multimodal")
        self._step_extras: dict = {}
        self.lora = None
        if cfg.lora.enable:
            from ..lora import LoRAManager
            self.lora = LoRAManager(self.model, cfg.lora.max_loras, cfg.lora.max_lora_rank, self.max_tokens, self.max_bs,
                                    self.device, self.model.dtype)
        self.sp_peer = None if self.lora is not None else self._init_sequence_parallel()
        self.attn_workspace = self._alloc_attn_workspace()
        self.last_tokens: Optional[torch.Tensor] = None  # previous step's sampled tokens (device)
        self.last_rows: dict = {}  # request_id -> row in last_tokens of its newest token
        self.kernel_launches = 0
        self.keep_full_hidden = False  # set by a proposer that needs every row's hidden state
        self._full_hidden = None
        if self.is_cuda and cfg.compilation.mode != "none":
            from ..compilation.cuda_graph import DecodeGraphs
            self.graphs = DecodeGraphs(self)

    # ------------------------------------------------------------------ memory
    @staticmethod
    def _layer_specs(spec):
        """A layer's cache spec is ``(shape_per_block, dtype)`` or a list of such pairs."""
        return spec if isinstance(spec, list) else [spec]

    def _bytes_per_block(self) -> int:
        total = 0
        for _, spec in self.model.kv_cache_spec(self.block_size).items():
            for shp, dt in self._layer_specs(spec):
                total += int(np.prod(shp)) * torch.empty((), dtype=dt).element_size()
        return total

    def _plan_num_blocks(self) -> int:
        if self.cfg.cache.num_blocks is not None:
            return self.cfg.cache.num_blocks
        per = max(1, self._bytes_per_block())
        if self.is_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            reserve = int(total * (1 - self.cfg.cache.gpu_memory_utilization))
            # activations for the largest step: a few [T, max(inter, vocab-shard)] buffers
            act = self.max_tokens * 16 * self.cfg.model.hidden_size * 2 + (2 << 30)
            budget = max(0, free - reserve - act)
            need = self.max_bs * self.max_blocks_per_seq
            n = int(max(16, min(budget // per, need + 64)))
            if torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
                # every rank must plan the same pool or the (replicated) schedulers would diverge
                t = torch.tensor([n], device=self.device, dtype=torch.int64)
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
                n = int(t.item())
            return n
        return min(self.max_bs * self.max_blocks_per_seq + 8, 4096)

    def _alloc_kv(self):
        caches = {}
        for i, spec in self.model.kv_cache_spec(self.block_size).items():
            ts = [torch.zeros((self.num_blocks, *shp), dtype=dt, device=self.device)
                  for shp, dt in self._layer_specs(spec)]
            caches[i] = ts[0] if not isinstance(spec, list) else tuple(ts)
        return caches

    def _init_sequence_parallel(self):
        """Fused GEMM+reduce-scatter / all-gather+GEMM path for large (prefill) steps under TP."""
        st = self.pstate
        m = self.cfg.model
        if (not self.is_cuda or st.tp_size == 1 or st.pp_size > 1 or st.tp_comm is None
                or st.tp_comm.peer is None or m.quantization is not None or self.model.dtype != torch.bfloat16):
            return None
        peer = st.tp_comm.peer
        peer.sp_init(self.max_tokens, m.hidden_size, self.model.dtype)
        from ..ops import gemm_cuda
        gemm_cuda.PEER = peer
        return peer

    def _alloc_attn_workspace(self):
        if not self.is_cuda or self.cfg.model.use_mla:
            return None
        from ..ops.attention_cuda import AttnWorkspace
        m = self.cfg.model
        heads = m.num_heads // self.pstate.tp_size
        return AttnWorkspace(self.max_bs * (1 + self.num_spec), heads, m.head_dim, 16, self.device)

    def _alloc_staging(self):
        T, B, MB = self.max_tokens, self.max_bs, self.max_blocks_per_seq
        pin = self.is_cuda
        self.n64 = 3 * T
        self.n32 = 2 * B + 2 + B * MB + T + T + 2 * B + 2 * T
        # Two staging sets used alternately: the host may fill step i+1 while the copies of step i
        # are still queued (the engine runs at most one step ahead of the device).
        self._h64s = [torch.zeros(self.n64, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self._h32s = [torch.zeros(self.n32, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.d64 = torch.zeros(self.n64, dtype=torch.int64, device=self.device)
        self.d32 = torch.zeros(self.n32, dtype=torch.int32, device=self.device)
        self._tok_hosts = [torch.zeros(max(T, B * (1 + self.num_spec)), dtype=torch.int64, pin_memory=pin)
                           for _ in range(2)]
        self._lp_hosts = [torch.zeros(max(T, B * (1 + self.num_spec)), dtype=torch.float32, pin_memory=pin)
                          for _ in range(2)]
        self._status_hosts = [torch.zeros(8, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._status_cache = None
        self.step_idx = 0
        self._bind_staging()
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _bind_staging(self):
        k = self.step_idx & 1
        self.h64, self.h32, self.tokens_host = self._h64s[k], self._h32s[k], self._tok_hosts[k]
        self.h64_np, self.h32_np = self.h64.numpy(), self.h32.numpy()

    # ------------------------------------------------------------------ multimodal
    def encode_multimodal(self, prompt_token_ids, data: dict) -> dict:
        """Run the vision tower for one request and work out which prompt rows its embeddings replace."""
        assert self.is_vl, "the loaded model has no vision tower"
        if hasattr(self.model, "encode_multimodal_data"):  # several modalities: the model sorts out its placeholders
            embeds, rows, pos3, delta = self.model.encode_multimodal_data(prompt_token_ids, data)
            return {"embeds": embeds, "rows": np.asarray(rows, dtype=np.int64),
                    "pos3": None if pos3 is None else pos3.numpy(), "delta": int(delta)}
        grid = data.get("image_grid_thw")
        grid = [tuple(int(x) for x in g) for g in (grid.tolist() if hasattr(grid, "tolist") else grid)] if grid is not None else None
        embeds = self.model.embed_multimodal(data["pixel_values"], grid)
        rows, pos3, delta = self.model.mm_metadata(prompt_token_ids, grid)
        assert len(rows) == embeds.shape[0], f"{len(rows)} image placeholder tokens but {embeds.shape[0]} image embeddings"
        return {"embeds": embeds, "rows": np.asarray(rows, dtype=np.int64), "pos3": None if pos3 is None else pos3.numpy(),
                "delta": int(delta)}

    def _prepare_multimodal(self, srs, pos, Tp):
        """Image-row overrides and 3-axis rotary positions for this step (prefill chunks that touch images)."""
        self._step_extras = {}
        dst, src = [], []
        pos3 = None
        t = 0
        for sr in srs:
            r, n, c = sr.req, sr.num_new_tokens, sr.req.num_computed_tokens
            if r.mm is not None:
                L = r.num_prompt_tokens
                if r.mm["delta"]:
                    hi = np.arange(c, c + n)
                    pos[t:t + n] = np.where(hi >= L, hi + r.mm["delta"], hi)
                rows = r.mm["rows"]
                sel = np.nonzero((rows >= c) & (rows < c + n))[0]
                if len(sel):
                    dst.append(torch.from_numpy(t + rows[sel] - c))
                    src.append(r.mm["embeds"].index_select(0, torch.from_numpy(sel).to(self.device)))
                if r.mm["pos3"] is not None and c < L:
                    if pos3 is None:
                        pos3 = np.repeat(pos[None, :Tp], 3, 0)
                    k = min(n, L - c)
                    pos3[:, t:t + k] = r.mm["pos3"][:, c:c + k]
            t += n
        if pos3 is not None:
            # rows filled after this request's turn still hold the 1-D positions written by the main loop
            t = 0
            for sr in srs:
                r, n, c = sr.req, sr.num_new_tokens, sr.req.num_computed_tokens
                if r.mm is None or r.mm["pos3"] is None or c >= r.num_prompt_tokens:
                    pos3[:, t:t + n] = pos[t:t + n]
                else:
                    k = min(n, r.num_prompt_tokens - c)
                    pos3[:, t + k:t + n] = pos[t + k:t + n]
                t += n
            self._step_extras["mrope_positions"] = torch.from_numpy(pos3.copy()).to(self.device, non_blocking=True)
        if dst:
            self._step_extras["mm_dst"] = torch.cat(dst).to(self.device, non_blocking=True)
            self._step_extras["mm_src"] = torch.cat(src)

    # ------------------------------------------------------------------ input preparation
    def prepare(self, sched: SchedulerOutput, pad_reqs: int = 0):
        """Fill the staging buffers for this step; returns ``(AttentionMetadata, input_ids, info)``."""
        bs = self.block_size
        srs = sched.scheduled
        B = len(srs)
        Bp = max(B, pad_reqs)
        T = sched.num_tokens
        Tp = T + (Bp - B)  # padded decode rows carry one dummy token each
        ids = self.h64_np[0:Tp]
        pos = self.h64_np[self.max_tokens:self.max_tokens + Tp]
        slots = self.h64_np[2 * self.max_tokens:2 * self.max_tokens + Tp]
        seq_lens = self.h32_np[0:Bp]
        qsl = self.h32_np[self.max_bs:self.max_bs + Bp + 1]
        o_bt = 2 * self.max_bs + 2
        max_seq = 0
        max_q = 0
        nblk = 1
        for sr in srs:
            nblk = max(nblk, len(sr.req.block_ids))
        nblk = min(self.max_blocks_per_seq, round_up(nblk, 8))
        if pad_reqs:
            nblk = self.max_blocks_per_seq  # graph buffers have a fixed row stride
        bt = self.h32_np[o_bt:o_bt + Bp * nblk].reshape(Bp, nblk)
        o_li = o_bt + self.max_bs * self.max_blocks_per_seq
        logits_idx = self.h32_np[o_li:o_li + self.max_tokens]
        o_rq = o_li + self.max_tokens
        req_of_tok = self.h32_np[o_rq:o_rq + Tp]
        o_ss = o_rq + self.max_tokens
        state_idx = self.h32_np[o_ss:o_ss + Bp]
        has_init = self.h32_np[o_ss + self.max_bs:o_ss + self.max_bs + Bp]
        o_lo = o_ss + 2 * self.max_bs
        lora_tok = self.h32_np[o_lo:o_lo + Tp]
        lora_row = self.h32_np[o_lo + self.max_tokens:o_lo + 2 * self.max_tokens]
        any_lora = False
        t = 0
        n_logits = 0
        sample_reqs, rows_per_req = [], []
        pending_dst, pending_src = [], []
        num_decodes = num_decode_tokens = 0
        qsl[0] = 0
        for b, sr in enumerate(srs):
            r, n = sr.req, sr.num_new_tokens
            c = r.num_computed_tokens
            known = r.all_token_ids
            n_spec = len(r.spec_token_ids) if sr.is_decode else 0
            n_known = n - n_spec
            chunk = known[c:c + n_known]
            if len(chunk) < n_known:  # newest token still on the device (async scheduling)
                assert len(chunk) == n_known - 1 and r.request_id in self.last_rows
                pending_dst.append(t + n_known - 1)
                pending_src.append(self.last_rows[r.request_id])
                chunk = chunk + [0]
            ids[t:t + n_known] = chunk
            if n_spec:
                ids[t + n_known:t + n] = r.spec_token_ids
            p = np.arange(c, c + n)
            pos[t:t + n] = p
            blocks = np.asarray(r.block_ids, dtype=np.int64)
            if self.dcp > 1:  # token p lives on rank p % dcp at local position p // dcp
                vb = bs * self.dcp
                slots[t:t + n] = np.where(p % self.dcp == self.dcp_rank, blocks[p // vb] * bs + (p % vb) // self.dcp, -1)
            else:
                slots[t:t + n] = blocks[p // bs] * bs + p % bs
            bt[b, :len(r.block_ids)] = r.block_ids
            bt[b, len(r.block_ids):] = 0
            seq_lens[b] = c + n
            qsl[b + 1] = t + n
            state_idx[b] = r.state_slot
            has_init[b] = 1 if c > 0 else 0
            lslot = self.lora.slot_for(r.lora_id) if self.lora is not None else -1
            any_lora |= lslot >= 0
            lora_tok[t:t + n] = lslot
            req_of_tok[t:t + n] = b
            max_seq = max(max_seq, c + n)
            max_q = max(max_q, n)
            if sr.is_decode:
                num_decodes += 1
                num_decode_tokens += n
            if sr.samples:
                rows = n if (sr.is_decode and n_spec) else 1
                logits_idx[n_logits:n_logits + rows] = np.arange(t + n - rows, t + n)
                lora_row[n_logits:n_logits + rows] = lslot
                n_logits += rows
                sample_reqs.append(r)
                rows_per_req.append(rows)
            t += n
        for b in range(B, Bp):  # padding rows for a captured batch size
            ids[t] = 0
            pos[t] = 0
            slots[t] = -1
            bt[b, :] = 0
            seq_lens[b] = 0
            qsl[b + 1] = t + 1
            state_idx[b] = -1
            has_init[b] = 0
            lora_tok[t] = -1
            lora_row[n_logits] = -1
            req_of_tok[t] = b
            logits_idx[n_logits] = t
            n_logits += 1
            t += 1
        if self.is_vl:
            self._prepare_multimodal(srs, pos, Tp)
        if pad_reqs:  # a padded (graph) batch is decode-shaped throughout
            num_decodes, num_decode_tokens = Bp, Tp
        # ---- host -> device
        if self.is_cuda:
            MT_ = self.max_tokens
            if Tp * 8 < MT_:  # small step: three short copies beat one long one
                for o in (0, MT_, 2 * MT_):
                    self.d64[o:o + Tp].copy_(self.h64[o:o + Tp], non_blocking=True)
            else:
                self.d64.copy_(self.h64, non_blocking=True)
            n32_used = o_rq + Tp
            self.d32[:n32_used].copy_(self.h32[:n32_used], non_blocking=True)
            if self.lora is not None:
                self.d32[o_lo:o_lo + Tp].copy_(self.h32[o_lo:o_lo + Tp], non_blocking=True)
                o_lr = o_lo + self.max_tokens
                self.d32[o_lr:o_lr + n_logits].copy_(self.h32[o_lr:o_lr + n_logits], non_blocking=True)
                self.h2d_bytes += 4 * (Tp + n_logits)
            if self.num_state_slots:
                self.d32[o_ss:o_ss + 2 * self.max_bs].copy_(self.h32[o_ss:o_ss + 2 * self.max_bs], non_blocking=True)
                self.h2d_bytes += 8 * self.max_bs
            self.h2d_bytes += Tp * 8 * 3 + (Bp * 2 + 1 + Bp * nblk + n_logits + Tp) * 4
            src64, src32 = self.d64, self.d32
        else:
            src64, src32 = self.h64.clone(), self.h32.clone()
        MT = self.max_tokens
        input_ids = src64[0:Tp]
        md = AttentionMetadata(
            num_tokens=Tp, num_reqs=Bp, positions=src64[MT:MT + Tp], slot_mapping=src64[2 * MT:2 * MT + Tp],
            block_tables=src32[o_bt:o_bt + Bp * nblk].view(Bp, nblk), seq_lens=src32[0:Bp],
            query_start_loc=src32[self.max_bs:self.max_bs + Bp + 1], max_query_len=max(max_q, 1),
            max_seq_len=max(max_seq, 1), num_decodes=num_decodes, num_decode_tokens=num_decode_tokens,
            num_prefills=Bp - num_decodes, workspace=self.attn_workspace, req_id_per_token=src32[o_rq:o_rq + Tp],
            logits_indices=src32[o_li:o_li + n_logits], num_spec_tokens=self.num_spec)
        if self.lora is not None:
            # a captured graph always runs the adapter kernels (ids of -1 make them no-ops)
            self.lora.punica.update_metadata(src32[o_lo:o_lo + Tp],
                                             src32[o_lo + self.max_tokens:o_lo + self.max_tokens + n_logits],
                                             no_lora=not any_lora and not pad_reqs)
        if self.num_state_slots:
            md.state_indices = src32[o_ss:o_ss + Bp]
            md.has_initial_state = src32[o_ss + self.max_bs:o_ss + self.max_bs + Bp]
        if not self.is_cuda:
            md.seq_lens_cpu, md.query_start_loc_cpu = md.seq_lens, md.query_start_loc
        else:
            md.seq_lens_cpu = torch.from_numpy(seq_lens.copy())
            md.query_start_loc_cpu = torch.from_numpy(qsl.copy())
        if pending_dst:
            dst = torch.tensor(pending_dst, dtype=torch.int64)
            src = torch.tensor(pending_src, dtype=torch.int64)
            if self.is_cuda:
                dst, src = dst.to(self.device, non_blocking=True), src.to(self.device, non_blocking=True)
            input_ids.index_copy_(0, dst, self.last_tokens.index_select(0, src))
        return md, input_ids, (sample_reqs, rows_per_req, n_logits)

    # ------------------------------------------------------------------ execution
    @torch.inference_mode()
    def execute(self, sched: SchedulerOutput) -> StepHandle:
        t0 = time.perf_counter()
        self.step_idx += 1
        self._bind_staging()
        srs = sched.scheduled
        use_graph = (self.graphs is not None and all(s.is_decode for s in srs)
                     and self.graphs.supports(len(srs), sched.num_tokens))
        pad = self.graphs.padded_batch(len(srs)) if use_graph else 0
        md, input_ids, (sample_reqs, rows_per_req, n_logits) = self.prepare(sched, pad)
        sp = self.sampler.make_params([r.sampling for r in sample_reqs], rows_per_req, n_logits, reqs=sample_reqs)
        from ..models.layers import set_sp_mode
        if use_graph:
            set_sp_mode(False)
            tokens, hidden = self.graphs.run(md, input_ids, sp)
        else:
            set_sp_mode(self.sp_peer is not None and md.num_tokens >= 128 * self.pstate.tp_size)
            try:
                tokens, hidden = self.forward_and_sample(md, input_ids, sp)
            finally:
                set_sp_mode(False)
        n_real = sum(rows_per_req)
        tokens = tokens[:n_real]
        # bookkeeping at launch time: the KV of these tokens is (being) written
        row = 0
        self.last_rows = {}
        for r, rows in zip(sample_reqs, rows_per_req):
            self.last_rows[r.request_id] = row + rows - 1
            row += rows
        for sr in srs:
            sr.req.num_computed_tokens += sr.num_new_tokens
        self.last_tokens = tokens
        ev = None
        lp_cpu = status_cpu = None
        names = ()
        lp = self.sampler.last_logprobs
        if self.is_cuda:
            tokens_cpu = self.tokens_host[:n_real]
            tokens_cpu.copy_(tokens, non_blocking=True)
            self.d2h_bytes += n_real * 8
            if lp is not None:
                lp_cpu = self._lp_hosts[self.step_idx & 1][:n_real]
                lp_cpu.copy_(lp[:n_real], non_blocking=True)
                self.d2h_bytes += n_real * 4
            words = self._status_words()
            if words:
                # the status words of every kernel family that waits on a peer or a barrier ride along with the
                # tokens, so a timed-out wait surfaces as an error of THIS step instead of as silently wrong tokens
                names = tuple(n for n, _ in words)
                status_cpu = self._status_hosts[self.step_idx & 1][:len(words)]
                for i, (_, w) in enumerate(words):
                    status_cpu[i:i + 1].copy_(w.view(-1)[:1], non_blocking=True)
                self.d2h_bytes += 4 * len(words)
            ev = torch.cuda.Event()
            ev.record()
        else:
            tokens_cpu = tokens
            lp_cpu = None if lp is None else lp[:n_real]
        full = None
        if self.keep_full_hidden:
            full = hidden if use_graph else self._full_hidden
        return StepHandle(sched, sample_reqs, rows_per_req, tokens, tokens_cpu, ev, hidden, t0, md, input_ids, full,
                          lp_cpu, status_cpu, names)

    def _status_words(self) -> list:
        """``(name, int32 device tensor)`` of every status word a kernel of this process may have set."""
        st = self.pstate
        a2a = getattr(st, "ep_a2a", None)
        if getattr(self, "_status_cache", None) is None or self._status_has_a2a != (a2a is not None):
            self._status_has_a2a = a2a is not None
            words = []
            for name, comm in (("tp", st.tp_comm), ("ep", getattr(st, "ep_comm", None)),
                               ("dcp", getattr(st, "dcp_comm", None))):
                peer = getattr(comm, "peer", None) if comm is not None else None
                if peer is not None and all(peer.status is not w for _, w in words):
                    words.append((f"{name}_peer", peer.status))
            if a2a is not None:  # expert dispatch / combine (created on first use)
                words.append(("ep_a2a", a2a.h.status_tensor()))
            from ..ops import _ext
            if _ext.available():
                gs = _ext.C().gemm_status_tensor()
                if gs is not None:
                    words.append(("gemm", gs))
            self._status_cache = words
        return self._status_cache

    def forward_and_sample(self, md: AttentionMetadata, input_ids, sp, capturing: bool = False):
        ctx = ForwardContext(attn=md, kv_caches=self.kv_caches, pstate=self.pstate, capturing=capturing,
                             lora=None if self.lora is None else self.lora.punica, extras=self._step_extras)
        with set_forward_context(ctx):
            hidden = self.run_model(input_ids, md)
            st = self.pstate
            if hidden is None:  # not the last pipeline stage: sampled ids arrive from the last one
                tokens = torch.zeros(md.logits_indices.shape[0], dtype=torch.int64, device=self.device)
                sel = None
            else:
                self._full_hidden = hidden if self.keep_full_hidden else None
                if self.keep_full_hidden and getattr(self.model, "aux_hidden", None) is not None:
                    self._full_hidden = self.model.aux_hidden  # EAGLE-3 drafts read three layers' states
                sel = hidden.index_select(0, md.logits_indices.long()) if md.logits_indices is not None else hidden
                logits = self.model.compute_logits(sel)
                tokens = self.sampler(logits, sp)
            if st.pp_size > 1:
                st.pp_comm.broadcast(tokens, src=st.pp_size - 1)
        return tokens, sel

    def run_model(self, input_ids, md):
        """One pipeline stage: receive from the previous stage, run, send on (NCCL p2p)."""
        st = self.pstate
        hidden = residual = None
        if st.pp_size > 1 and not st.is_first_pp:
            shape = (md.num_tokens, self.cfg.model.hidden_size)
            hidden = st.pp_comm.recv(shape, self.model.dtype, st.pp_rank - 1)
            residual = st.pp_comm.recv(shape, self.model.dtype, st.pp_rank - 1)
        hidden, residual = self.model(input_ids, hidden, residual)
        if st.pp_size > 1 and not st.is_last_pp:
            st.pp_comm.isend_side_stream(hidden, st.pp_rank + 1)
            st.pp_comm.isend_side_stream(residual, st.pp_rank + 1)
            return None
        return hidden

    def profile_run(self, num_tokens: int):
        """Dummy forward to size activations (``attn_metadata is None`` path of the reference,
        ``kunlun_attn.py:770-772``)."""
        from .request import Request, SamplingParams
        from .scheduler import ScheduledRequest
        n = max(1, min(num_tokens, self.max_tokens))
        req = Request("profile-run", [1] * n, SamplingParams(max_tokens=1))
        req.block_ids = [0] * cdiv(n, self.tokens_per_block)
        if self.num_state_slots:
            req.state_slot = 0
        sched = SchedulerOutput(scheduled=[ScheduledRequest(req, n, False, True)], num_tokens=n)
        self.step_idx += 1
        self._bind_staging()
        with torch.inference_mode():
            md, ids, (sample_reqs, rows, n_logits) = self.prepare(sched)
            md.slot_mapping.fill_(-1)  # nothing is written to the cache
            md.is_dummy = True
            sp = self.sampler.make_params([req.sampling], rows, n_logits)
            if self.is_cuda:
                torch.cuda.synchronize()
                torch.cuda.reset_peak_memory_stats(self.device)
            self.forward_and_sample(md, ids, sp)
            if self.is_cuda:
                torch.cuda.synchronize()
                return int(torch.cuda.max_memory_allocated(self.device))
        return 0
