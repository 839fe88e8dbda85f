"""Token sampler: greedy, temperature, top-k / top-p, repetition penalty - no host synchronisation.

Behaviour follows ``TopKTopPSampler`` of the reference (``v1/sample/ops/topk_topp_sampler.py:51-216``):
greedy rows take the argmax, random rows scale by temperature, mask by top-k / top-p, soft-max and
draw by the exponential race ``argmax(p / Exp(1))`` (``:141-174``).  All per-request parameters
travel as device tensors, so the sampler can sit inside a captured CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops.reference import misc as ref


@dataclass
class SamplingTensors:
    all_greedy: bool
    temperature: Optional[torch.Tensor] = None  # [n] fp32
    top_k: Optional[torch.Tensor] = None  # [n] int32 (0 = off) or None
    top_p: Optional[torch.Tensor] = None  # [n] fp32 or None
    n: int = 0
    # repetition penalty: rows with a penalty != 1 scale the logits of every token seen so far
    penalties: Optional[torch.Tensor] = None  # [n] fp32
    history: Optional[torch.Tensor] = None    # [n, L] int64 prompt + output tokens (padded with -1)
    history_len: Optional[torch.Tensor] = None  # [n] int32
    # per-request seeds: rows with a seed draw their Exp(1) noise from their own generator
    seeded: Optional[list] = None             # [(row, seed, draw index)]
    want_logprobs: bool = False


class Sampler:
    def __init__(self, vocab_size: int, device, seed: int = 0):
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.seed = seed
        self.last_logprobs: Optional[torch.Tensor] = None  # log p(sampled token) of the last call, when asked for

    def make_params(self, params: list, rows_per_req: list, n_rows: int, reqs: Optional[list] = None) -> SamplingTensors:
        """``reqs`` (the requests behind ``params``, same order) supplies the token history for repetition
        penalties and the draw counter for per-request seeds."""
        want_lp = any(p.logprobs for p in params)
        need_pen = reqs is not None and any(p.repetition_penalty != 1.0 for p in params)
        if all(p.greedy for p in params) and not need_pen:
            return SamplingTensors(all_greedy=True, n=n_rows, want_logprobs=want_lp)
        temps, ks, ps, pens = [], [], [], []
        for p, rows in zip(params, rows_per_req):
            temps += [p.temperature] * rows
            ks += [p.top_k] * rows
            ps += [p.top_p] * rows
            pens += [p.repetition_penalty] * rows
        pad = n_rows - len(temps)
        temps += [0.0] * pad
        ks += [0] * pad
        ps += [1.0] * pad
        pens += [1.0] * pad
        dev = self.device
        out = SamplingTensors(
            all_greedy=all(t == 0.0 for t in temps),
            temperature=torch.tensor(temps, dtype=torch.float32).to(dev, non_blocking=True),
            top_k=torch.tensor(ks, dtype=torch.int32).to(dev, non_blocking=True) if any(ks) else None,
            top_p=torch.tensor(ps, dtype=torch.float32).to(dev, non_blocking=True) if any(x < 1 for x in ps) else None,
            n=n_rows, want_logprobs=want_lp)
        if need_pen:
            hist, lens = [], []
            for r, rows in zip(reqs, rows_per_req):
                toks = r.all_token_ids if r.sampling.repetition_penalty != 1.0 else []
                hist += [toks] * rows
                lens += [len(toks)] * rows
            hist += [[]] * pad
            lens += [0] * pad
            L = max(1, max(lens))
            h = torch.full((n_rows, L), -1, dtype=torch.int64)
            for i, toks in enumerate(hist):
                if toks:
                    h[i, :len(toks)] = torch.tensor(toks, dtype=torch.int64)
            out.penalties = torch.tensor(pens, dtype=torch.float32).to(dev, non_blocking=True)
            out.history = h.to(dev, non_blocking=True)
            out.history_len = torch.tensor(lens, dtype=torch.int32).to(dev, non_blocking=True)
        if reqs is not None and any(p.seed is not None and not p.greedy for p in params):
            out.seeded, row = [], 0
            for r, rows in zip(reqs, rows_per_req):
                if r.sampling.seed is not None and not r.sampling.greedy:
                    out.seeded += [(row + j, int(r.sampling.seed), len(r.output_token_ids) + r.num_pending + j)
                                   for j in range(rows)]
                row += rows
        return out

    def _seeded_noise(self, logits, seeded):
        """Exp(1) noise for every row; seeded rows draw from ``Generator(seed)`` advanced to their draw index, so a
        request with a seed reproduces its tokens whatever else is in the batch."""
        q = torch.empty(logits.shape, dtype=torch.float32, device=logits.device).exponential_(generator=self.gen)
        for row, seed, draw in seeded:
            g = torch.Generator(device=logits.device)
            g.manual_seed((seed * 1000003 + draw) & 0x7FFFFFFFFFFFFFFF)
            q[row] = torch.empty(logits.shape[1], dtype=torch.float32, device=logits.device).exponential_(generator=g)
        return q

    def __call__(self, logits: torch.Tensor, sp: SamplingTensors) -> torch.Tensor:
        self.last_logprobs = None
        if sp.penalties is not None:
            logits = ops.apply_repetition_penalty(logits.float() if not logits.is_cuda else logits, sp.history,
                                                  sp.history_len, sp.penalties)
        if sp.all_greedy:
            tokens = ops.argmax(logits)
        else:
            q = self._seeded_noise(logits, sp.seeded) if sp.seeded else None
            tokens = self.sample(logits, sp.temperature, sp.top_k, sp.top_p, q=q)
        if sp.want_logprobs:
            self.last_logprobs = logits.float().log_softmax(-1).gather(1, tokens.view(-1, 1)).squeeze(1)
        return tokens

    def sample(self, logits, temperature, top_k=None, top_p=None, q=None):
        if logits.is_cuda:
            # one launch: temperature, radix-select top-k / top-p thresholds, exponential race
            return ops.topk_topp_sample(logits, temperature, top_k, top_p, noise=q, seed=self.seed)
        greedy = ops.argmax(logits)
        t = temperature
        lg = logits.float() / torch.where(t == 0, torch.ones_like(t), t).unsqueeze(1)
        if top_k is not None:
            V = lg.shape[-1]
            top_k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k)
        lg = ref.apply_top_k_top_p(lg, top_k, top_p) if not lg.is_cuda else _mask_top_k_top_p_cuda(lg, top_k, top_p)
        probs = lg.softmax(-1)
        if q is None:
            q = torch.empty_like(probs).exponential_(generator=self.gen)
        rnd = (probs / q).argmax(-1)
        return torch.where(t == 0, greedy, rnd)

    def probs(self, logits, temperature, top_k=None, top_p=None):
        """Post-processing distribution (used by the rejection sampler)."""
        t = temperature
        lg = logits.float() / torch.where(t == 0, torch.ones_like(t), t).unsqueeze(1)
        if top_k is not None:
            top_k = torch.where(top_k <= 0, torch.full_like(top_k, lg.shape[-1]), top_k)
        lg = ref.apply_top_k_top_p(lg, top_k, top_p) if not lg.is_cuda else _mask_top_k_top_p_cuda(lg, top_k, top_p)
        return lg.softmax(-1)


def _mask_top_k_top_p_cuda(lg, top_k, top_p):
    """Device path: same sort-based masking with torch primitives (vocab-wide sort per row).  The
    rejection-style sampling kernel replaces it when available."""
    if top_k is None and top_p is None:
        return lg
    return ref.apply_top_k_top_p(lg, top_k, top_p)
