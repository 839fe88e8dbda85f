"""CUDA-graph capture and replay of decode steps.

The reference supports piecewise graphs only: the model is split at the attention op, each piece is
captured, and attention runs eagerly between pieces, one host launch sequence per layer
(``docs/source/developer_guide/feature_guide/Kunlun_Graph.md:58-75``; platform hooks
``platforms/kunlun.py:100-106,366-378``).  The attention kernels here read all per-step state from
device tensors at fixed addresses (block tables, lengths, slot mapping live in the runner's
persistent staging buffers), so a whole decode step - embedding to logits - is captured as ONE graph
per padded batch size and replayed with no per-layer host work.
"""
from __future__ import annotations

import bisect
from typing import Optional

import torch

from ..attention.metadata import AttentionMetadata


class DecodeGraphs:
    def __init__(self, runner):
        self.runner = runner
        cfg = runner.cfg
        self.tokens_per_req = 1 + cfg.speculative.num_speculative_tokens
        self.sizes = sorted(s for s in cfg.compilation.capture_sizes if s <= runner.max_bs)
        if runner.max_bs not in self.sizes and runner.max_bs <= 512:
            self.sizes.append(runner.max_bs)
        self.graphs: dict = {}
        self.logits: dict = {}
        self.hidden: dict = {}
        self.pool = None
        self.hits = 0
        self.kernels_per_graph: dict = {}
        self.replayed_kernels = 0
        self.misses = 0
        from .. import envs
        self.watcher = None
        if envs.B200_GRAPH_WATCH:
            from ..utils.hooks import GraphInputWatcher
            self.watcher = GraphInputWatcher()

    def supports(self, num_reqs: int, num_tokens: int) -> bool:
        ok = (num_reqs > 0 and num_tokens == num_reqs * self.tokens_per_req and self.sizes
              and num_reqs <= self.sizes[-1])
        if not ok:
            self.misses += 1
        return bool(ok)

    def padded_batch(self, num_reqs: int) -> int:
        return self.sizes[bisect.bisect_left(self.sizes, num_reqs)]

    def _forward(self, md: AttentionMetadata, input_ids):
        from ..attention.metadata import ForwardContext, set_forward_context
        r = self.runner
        ctx = ForwardContext(attn=md, kv_caches=r.kv_caches, pstate=r.pstate, capturing=True,
                             lora=None if r.lora is None else r.lora.punica)
        with set_forward_context(ctx):
            hidden = r.run_model(input_ids, md)
            sel = hidden.index_select(0, md.logits_indices.long())
            return r.model.compute_logits(sel), sel

    def _capture(self, md: AttentionMetadata, input_ids):
        key = md.num_reqs
        # plan attention splits for the longest context this graph may ever see
        md.max_seq_len = self.runner.cfg.scheduler.max_model_len
        md.max_query_len = self.tokens_per_req
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):  # warm-up: lazy allocations, tensor-map cache, function attributes
                self._forward(md, input_ids)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        from ..ops import _ext
        g = torch.cuda.CUDAGraph()
        n0 = _ext.C().launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            logits, sel = self._forward(md, input_ids)
        self.kernels_per_graph[key] = _ext.C().launch_count() - n0
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[key], self.logits[key], self.hidden[key] = g, logits, sel
        if self.watcher is not None:
            self.watcher.capture(str(key), self._watched(md, input_ids))
        self._rendezvous()

    @staticmethod
    def _rendezvous():
        """Ranks capture the same graph at the same step, but a capture of a deep model takes seconds and not the
        same time everywhere; without this the first replay of the fastest rank would sit in its first peer wait
        for the difference."""
        import torch.distributed as dist

        from ..parallel.state import get_state
        if not (dist.is_available() and dist.is_initialized()):
            return
        st = get_state()
        # only the ranks of this model replica meet (tensor- and pipeline-parallel peers): data-parallel replicas
        # schedule independently and may capture at different times
        groups = [g for g, n in ((st.tp_group, st.tp_size), (st.pp_group, st.pp_size)) if g is not None and n > 1]
        if not groups:
            return
        torch.cuda.synchronize()
        for g in groups:
            if dist.get_backend(g) == "nccl":
                dist.barrier(group=g, device_ids=[torch.cuda.current_device()])
            else:
                dist.barrier(group=g)

    @torch.inference_mode()
    def run(self, md: AttentionMetadata, input_ids, sp):
        key = md.num_reqs
        if key not in self.graphs:
            self._capture(md, input_ids)
        self.hits += 1
        if self.watcher is not None:  # debug aid: a replay must see its inputs at the captured addresses
            self.watcher.check(str(key), self._watched(md, input_ids))
        self.graphs[key].replay()
        self.replayed_kernels += self.kernels_per_graph[key]
        tokens = self.runner.sampler(self.logits[key], sp)
        return tokens, self.hidden[key]

    @staticmethod
    def _watched(md, input_ids) -> dict:
        return {"input_ids": input_ids, "positions": md.positions, "slot_mapping": md.slot_mapping,
                "block_tables": md.block_tables, "seq_lens": md.seq_lens, "query_start_loc": md.query_start_loc,
                "logits_indices": md.logits_indices}

    def capture_all(self):
        """Eagerly capture every configured size with a synthetic decode batch (server warm-up), so that the first
        real request of each size does not pay for the capture."""
        from ..engine.request import Request, SamplingParams
        from ..engine.scheduler import ScheduledRequest, SchedulerOutput
        r = self.runner
        done = []
        with torch.inference_mode():
            for size in self.sizes:
                if size in self.graphs:
                    continue
                reqs = []
                for i in range(size):
                    q = Request(f"warmup-{size}-{i}", [1] * self.tokens_per_req, SamplingParams(max_tokens=1))
                    q.block_ids = [0]
                    q.num_computed_tokens = 0
                    reqs.append(ScheduledRequest(q, self.tokens_per_req, True, True))
                    if self.tokens_per_req > 1:
                        q.prompt_token_ids, q.spec_token_ids = [1], [1] * (self.tokens_per_req - 1)
                sched = SchedulerOutput(scheduled=reqs, num_tokens=size * self.tokens_per_req)
                r.step_idx += 1
                r._bind_staging()
                md, ids, _ = r.prepare(sched, size)
                md.slot_mapping.fill_(-1)  # synthetic tokens must not touch the cache
                self._capture(md, ids)
                done.append(size)
            torch.cuda.synchronize()
        return done
