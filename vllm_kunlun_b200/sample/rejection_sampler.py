"""Vectorised rejection sampler for speculative decoding - no host synchronisation, no Python loops.

The reference ports upstream's Triton kernels to PyTorch and falls back to Python double loops with
``.item()`` per token for the random path (``v1/sample/rejection_sampler.py:524-574,602-641``), a known
host bottleneck.  Here every path is a handful of batched tensor ops on a padded ``[B, S]`` layout:

* greedy rows accept drafts while they equal the target arg-max and emit the arg-max at the first
  mismatch (``:439-521``);
* random rows accept draft ``x`` with probability ``min(1, p_target(x) / p_draft(x))`` and otherwise emit a
  token from the recovered distribution ``max(p_target - p_draft, 0)`` (exponential race);
* when every draft is accepted the bonus token is appended.
Output ``[B, S + 1]`` padded with ``-1``."""
from __future__ import annotations

from typing import Optional

import torch

PLACEHOLDER_TOKEN_ID = -1


class RejectionSampler:
    def __init__(self, generator: Optional[torch.Generator] = None):
        self.generator = generator

    def forward(self, draft_token_ids: torch.Tensor, num_draft: torch.Tensor, target_probs: torch.Tensor,
                bonus_token_ids: torch.Tensor, is_greedy: torch.Tensor, draft_probs: Optional[torch.Tensor] = None,
                uniform: Optional[torch.Tensor] = None, recover_q: Optional[torch.Tensor] = None,
                max_spec_len: Optional[int] = None) -> torch.Tensor:
        """``draft_token_ids [n]`` flattened, ``num_draft [B]``, ``target_probs [n, V]``,
        ``bonus_token_ids [B]``, ``is_greedy [B]`` bool."""
        dev = target_probs.device
        B = num_draft.shape[0]
        n, V = target_probs.shape
        S = int(max_spec_len) if max_spec_len is not None else int(num_draft.max().item()) if B else 0
        cu = torch.zeros(B + 1, dtype=torch.long, device=dev)
        cu[1:] = num_draft.long().cumsum(0)
        # padded [B, S] views of the flat per-draft data
        pos = torch.arange(S, device=dev).unsqueeze(0).expand(B, S)
        valid = pos < num_draft.long().unsqueeze(1)
        flat = (cu[:-1].unsqueeze(1) + pos).clamp(max=max(n - 1, 0))
        draft = torch.where(valid, draft_token_ids.long()[flat], torch.zeros_like(flat))
        tgt_argmax = target_probs.argmax(-1)[flat]
        p_t = target_probs[flat, draft]
        p_d = torch.ones_like(p_t) if draft_probs is None else draft_probs[flat, draft]
        if uniform is None:
            uniform = torch.rand(n, device=dev, generator=self.generator, dtype=torch.float32)
        u = uniform.float()[flat]
        greedy = is_greedy.bool().unsqueeze(1)
        accept = torch.where(greedy, tgt_argmax == draft, (p_d > 0) & (p_t / p_d.clamp(min=1e-30) >= u)) & valid
        # number of leading accepted drafts per request
        acc_prefix = accept.long().cumprod(1)
        n_acc = acc_prefix.sum(1)
        out = torch.full((B, S + 1), PLACEHOLDER_TOKEN_ID, dtype=torch.long, device=dev)
        keep = pos < n_acc.unsqueeze(1)
        out[:, :S] = torch.where(keep, draft, out[:, :S])
        # the token emitted at the first rejected position (if any)
        rejected = n_acc < num_draft.long()
        rej_pos = n_acc.clamp(max=max(S - 1, 0))
        if S > 0:
            rflat = flat.gather(1, rej_pos.unsqueeze(1)).squeeze(1)
            tp = target_probs[rflat].float()
            rdraft = draft.gather(1, rej_pos.unsqueeze(1)).squeeze(1)
            if draft_probs is None:
                adj = tp.clone()
                adj.scatter_(1, rdraft.unsqueeze(1), 0.0)
            else:
                adj = (tp - draft_probs[rflat].float()).clamp(min=0)
            q = recover_q.float() if recover_q is not None else torch.empty_like(adj).exponential_(generator=self.generator)
            recovered = (adj / q).argmax(-1)
            tok = torch.where(is_greedy.bool(), tgt_argmax.gather(1, rej_pos.unsqueeze(1)).squeeze(1), recovered)
            out.scatter_(1, rej_pos.unsqueeze(1), torch.where(rejected, tok, out.gather(1, rej_pos.unsqueeze(1)).squeeze(1)).unsqueeze(1))
        # bonus token when everything was accepted
        bonus_pos = num_draft.long().unsqueeze(1)
        cur = out.gather(1, bonus_pos).squeeze(1)
        out.scatter_(1, bonus_pos, torch.where(rejected, cur, bonus_token_ids.long()).unsqueeze(1))
        return out

    @staticmethod
    def parse_output(out: torch.Tensor) -> list:
        return [[t for t in row if t != PLACEHOLDER_TOKEN_ID] for row in out.tolist()]
