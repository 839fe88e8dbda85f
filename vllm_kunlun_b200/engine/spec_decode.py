"""Speculative decoding: proposers and the accept / roll-back logic of the engine.

Reference: ``v1/sample/spec_decode/eagle.py`` (``propose`` ``:22-252`` handles ``method == "mtp"``, shifts
the input ids, inserts the newly sampled tokens and runs the draft model) and the spec-as-decode
convention of the attention builders (``kunlun_attn.py:482-507``: a request with drafts is a decode
request with ``q_len = 1 + num_spec``).

Verification emits the TARGET's own sample at every position and accepts a draft while it equals that
sample - exact for greedy decoding and distribution-preserving for random sampling.  After a step the
request's ``num_computed_tokens`` is rolled back to the last accepted position, so rejected drafts'
KV entries are simply overwritten later."""
from __future__ import annotations

from typing import Optional

import torch

from ..attention.metadata import ForwardContext, set_forward_context


class NgramProposer:
    """Prompt-lookup drafts: continue the longest earlier occurrence of the last ``n`` tokens."""

    def __init__(self, engine, k: int, n: int = 3):
        self.k, self.n = k, n

    def accept(self, req, vals, stats):
        return _accept(req, vals, stats)

    def propose(self, handle, stats):
        for req in handle.sample_reqs:
            if req.status.finished:
                continue
            toks = req.all_token_ids
            req.spec_token_ids = []
            for n in range(min(self.n, len(toks) - 1), 0, -1):
                tail = toks[-n:]
                for s in range(len(toks) - n - 1, -1, -1):
                    if toks[s:s + n] == tail:
                        req.spec_token_ids = toks[s + n:s + n + self.k]
                        break
                if req.spec_token_ids:
                    break


def _accept(req, vals, stats):
    """``vals`` = target samples at the ``1 + k`` fed positions.  Returns the tokens to append."""
    drafts = req.spec_token_ids
    a = 0
    while a < len(drafts) and a < len(vals) - 1 and vals[a] == drafts[a]:
        a += 1
    stats["spec_proposed"] += len(drafts)
    stats["spec_accepted"] += a
    # roll the KV position back to the last accepted token (rejected drafts' KV will be rewritten)
    req.num_computed_tokens -= len(drafts) - a
    req.spec_token_ids = []
    req._accepted_rows = a  # row offset (within this step's rows) whose output is the newest token
    return vals[:a + 1]


class MTPProposer:
    """A draft model that reads the target's hidden states: one draft token per step.  MTP (the configuration
    the benchmark names) by default; :class:`EagleProposer` swaps the draft network."""

    def build_model(self, engine):
        from ..models.deepseek_mtp import DeepSeekMTP
        cfg = engine.cfg
        return DeepSeekMTP(cfg.model, device=cfg.device, target=engine.runner.model)

    def __init__(self, engine):
        self.engine = engine
        r = engine.runner
        cfg = engine.cfg
        assert cfg.speculative.num_speculative_tokens == 1, "the draft-model proposers draft one token per step"
        with torch.inference_mode():
            self.model = self.build_model(engine)
            if cfg.speculative.draft_weights_path:
                from ..models.loader import load_safetensors
                self.model.load_weights(load_safetensors(cfg.speculative.draft_weights_path))
            else:
                self.model.init_random(cfg.seed)
        # the draft layer's KV cache uses the target's block ids
        for i, spec in self.model.kv_cache_spec(r.block_size).items():
            specs = spec if isinstance(spec, list) else [spec]
            ts = [torch.zeros((r.num_blocks, *shp), dtype=dt, device=r.device) for shp, dt in specs]
            r.kv_caches[i] = tuple(ts) if isinstance(spec, list) else ts[0]
        r.keep_full_hidden = True

    def accept(self, req, vals, stats):
        return _accept(req, vals, stats)

    @torch.inference_mode()
    def propose(self, handle, stats):
        r = self.engine.runner
        md, full_hidden = handle.md, handle.full_hidden
        if md is None or full_hidden is None:
            return
        # shifted ids: row i of a request carries token i+1; the row whose target output is the
        # request's newest token carries that token
        ids = handle.input_ids
        qsl = md.query_start_loc_cpu.tolist()
        shifted = torch.zeros_like(ids)
        shifted[:-1] = ids[1:]
        fix_rows, fix_toks, draft_rows, reqs = [], [], [], []
        for b, sr in enumerate(handle.sched.scheduled):
            req = sr.req
            s, e = qsl[b], qsl[b + 1]
            if not sr.samples:
                # partial prompt chunk: the next prompt token is known
                fix_rows.append(e - 1)
                fix_toks.append(req.all_token_ids[min(req.num_computed_tokens, req.num_tokens - 1)])
                continue
            if req.status.finished or not req.output_token_ids:
                continue
            off = getattr(req, "_accepted_rows", None)
            row = (e - 1) if off is None else min(e - 1, s + off)
            req._accepted_rows = None
            fix_rows.append(row)
            fix_toks.append(req.output_token_ids[-1])
            draft_rows.append(row)
            reqs.append(req)
        if not reqs:
            return
        dev = r.device
        shifted[torch.tensor(fix_rows, dtype=torch.long, device=dev)] = torch.tensor(fix_toks, dtype=ids.dtype, device=dev)
        rows_t = torch.tensor(draft_rows, dtype=torch.long, device=dev)
        ctx = ForwardContext(attn=md, kv_caches=r.kv_caches, pstate=r.pstate)
        with set_forward_context(ctx):
            h = self.model(shifted, full_hidden)
            logits = self.model.compute_logits(h.index_select(0, rows_t))
        drafts = logits.float().argmax(-1).tolist()
        for req, d in zip(reqs, drafts):
            req.spec_token_ids = [int(d)]


class EagleProposer(MTPProposer):
    """EAGLE / EAGLE-3 drafts (``v1/sample/spec_decode/eagle.py:22-252``).  For EAGLE-3 the target collects the
    hidden states of three layers and the runner hands their concatenation to the draft."""

    def build_model(self, engine):
        from ..models.eagle import EagleDraftModel
        cfg = engine.cfg
        eagle3 = cfg.speculative.method == "eagle3"
        target = engine.runner.model
        if eagle3:
            assert hasattr(target, "set_aux_hidden_state_layers"), "the target model does not expose auxiliary hidden states"
            target.set_aux_hidden_state_layers(target.get_eagle3_aux_hidden_state_layers())
        return EagleDraftModel(cfg.model, device=cfg.device, target=target, eagle3=eagle3)


def build_proposer(engine):
    sc = engine.cfg.speculative
    if sc.method == "mtp":
        return MTPProposer(engine)
    if sc.method in ("eagle", "eagle3"):
        return EagleProposer(engine)
    if sc.method == "ngram":
        return NgramProposer(engine, sc.num_speculative_tokens, sc.ngram_n)
    raise ValueError(f"unsupported speculative method {sc.method!r} (mtp, eagle, eagle3, ngram)")
