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


class Sampler:
    def __init__(self, vocab_size: int, device, seed: int = 0):
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.seed = seed

    def make_params(self, params: list, rows_per_req: list, n_rows: int) -> SamplingTensors:
        if all(p.greedy for p in params):
            return SamplingTensors(all_greedy=True, n=n_rows)
        temps, ks, ps = [], [], []
        for p, rows in zip(params, rows_per_req):
            temps += [p.temperature] * rows
            ks += [p.top_k] * rows
            ps += [p.top_p] * rows
        pad = n_rows - len(temps)
        temps += [0.0] * pad
        ks += [0] * pad
        ps += [1.0] * pad
        dev = self.device
        return SamplingTensors(
            all_greedy=False,
            temperature=torch.tensor(temps, dtype=torch.float32).to(dev, non_blocking=True),
            top_k=torch.tensor(ks, dtype=torch.int32).to(dev, non_blocking=True) if any(ks) else None,
            top_p=torch.tensor(ps, dtype=torch.float32).to(dev, non_blocking=True) if any(x < 1 for x in ps) else None,
            n=n_rows)

    def __call__(self, logits: torch.Tensor, sp: SamplingTensors) -> torch.Tensor:
        if sp.all_greedy:
            return ops.argmax(logits)
        return self.sample(logits, sp.temperature, sp.top_k, sp.top_p)

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
