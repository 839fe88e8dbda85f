"""Paged-KV block pool and the continuous-batching scheduler.

Policy: running requests first (decode, or verify of ``1 + num_spec`` tokens), then waiting requests'
prefill chunks within the token budget; the batch is ordered decode-first, as the reference's
attention builder re-orders it (``v1/attention/backends/kunlun_attn.py:509-546``).  When the pool
runs dry the most recently admitted running request is preempted and recomputed later.
"""
from __future__ import annotations

import collections
import hashlib
from dataclasses import dataclass, field
from typing import Optional

from ..config import cdiv
from .request import Request, RequestStatus


class BlockPool:
    """Free-list allocator with optional hash-based prefix reuse (ref-counted blocks)."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = False):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.free = collections.deque(range(num_blocks))
        self.ref = [0] * num_blocks
        self.enable_prefix_caching = enable_prefix_caching
        self.hash_to_block: dict = {}
        self.block_hash: dict = {}
        self.evictable: "collections.OrderedDict[int, None]" = collections.OrderedDict()

    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.evictable)

    def _pop(self) -> int:
        if self.free:
            return self.free.popleft()
        b, _ = self.evictable.popitem(last=False)  # LRU cached block
        h = self.block_hash.pop(b, None)
        if h is not None:
            self.hash_to_block.pop(h, None)
        return b

    def allocate(self, n: int) -> Optional[list]:
        if n > self.num_free:
            return None
        out = []
        for _ in range(n):
            b = self._pop()
            self.ref[b] = 1
            out.append(b)
        return out

    def release(self, blocks) -> None:
        for b in reversed(blocks):
            self.ref[b] -= 1
            if self.ref[b] == 0:
                if b in self.block_hash:
                    self.evictable[b] = None
                else:
                    self.free.append(b)

    # ---- prefix caching ----
    @staticmethod
    def chain_hash(prev: bytes, tokens) -> bytes:
        return hashlib.blake2b(prev + b"|" + ",".join(map(str, tokens)).encode(), digest_size=16).digest()

    def match_prefix(self, token_ids, salt: bytes = b"") -> list:
        """Longest run of full cached blocks for this prompt (never the whole prompt).  ``salt`` seeds the hash
        chain with everything besides token ids that decides the KV contents: the LoRA adapter and a digest of the
        multimodal inputs (upstream mixes the lora id and the mm hashes into its block hash the same way)."""
        if not self.enable_prefix_caching:
            return []
        out, h = [], salt
        bs = self.block_size
        for i in range((len(token_ids) - 1) // bs):
            h = self.chain_hash(h, token_ids[i * bs:(i + 1) * bs])
            b = self.hash_to_block.get(h)
            if b is None:
                break
            out.append(b)
        for b in out:
            if self.ref[b] == 0:
                self.evictable.pop(b, None)
            self.ref[b] += 1
        return out

    def register_full_blocks(self, req: Request) -> None:
        if not self.enable_prefix_caching:
            return
        bs = self.block_size
        toks = req.all_token_ids
        h = req.cache_salt
        for i in range(min(req.num_computed_tokens // bs, len(req.block_ids))):
            h = self.chain_hash(h, toks[i * bs:(i + 1) * bs])
            b = req.block_ids[i]
            if b not in self.block_hash and h not in self.hash_to_block:
                self.block_hash[b] = h
                self.hash_to_block[h] = b


@dataclass
class ScheduledRequest:
    req: Request
    num_new_tokens: int  # tokens fed this step (prefill chunk, or 1 + drafts)
    is_decode: bool
    samples: bool  # logits wanted for this request this step


@dataclass
class SchedulerOutput:
    scheduled: list = field(default_factory=list)
    num_tokens: int = 0
    preempted: list = field(default_factory=list)

    @property
    def empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, pool: BlockPool, max_num_seqs: int, max_num_batched_tokens: int, max_model_len: int,
                 chunked_prefill: bool = True, num_spec_tokens: int = 0, num_state_slots: int = 0):
        self.pool = pool
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.chunked_prefill = chunked_prefill
        self.num_spec_tokens = num_spec_tokens
        self.waiting: "collections.deque[Request]" = collections.deque()
        self.running: list = []
        self.finished: list = []
        self.free_state_slots = list(range(num_state_slots))
        self.uses_state = num_state_slots > 0

    def add(self, req: Request) -> None:
        if req.num_prompt_tokens + req.sampling.max_tokens > self.max_model_len:
            req.sampling.max_tokens = max(1, self.max_model_len - req.num_prompt_tokens)
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _ensure_blocks(self, req: Request, total_tokens: int) -> bool:
        need = cdiv(total_tokens, self.pool.block_size) - len(req.block_ids)
        if need <= 0:
            return True
        got = self.pool.allocate(need)
        if got is None:
            return False
        req.block_ids.extend(got)
        return True

    def _preempt(self, req: Request) -> None:
        self.pool.release(req.block_ids)
        req.block_ids = []
        req.num_computed_tokens = 0
        req.spec_token_ids = []
        req.status = RequestStatus.PREEMPTED
        req.num_preemptions += 1
        if req.state_slot >= 0:
            self.free_state_slots.append(req.state_slot)
            req.state_slot = -1
        self.waiting.appendleft(req)

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.max_tokens
        decodes, prefills = [], []
        # 1) running requests
        i = 0
        while i < len(self.running):
            req = self.running[i]
            remaining = req.num_tokens + req.num_pending - req.num_computed_tokens
            if remaining > 1:  # prompt chunk, or recompute after preemption
                n = min(remaining, budget) if self.chunked_prefill else remaining
                if n <= 0 or n > budget:
                    i += 1
                    continue
                is_decode = False
            else:
                # drafts must not run past the last position the model may see
                room = self.max_model_len - req.num_computed_tokens - 1
                if len(req.spec_token_ids) > max(0, room):
                    req.spec_token_ids = req.spec_token_ids[:max(0, room)]
                n = 1 + len(req.spec_token_ids)
                if n > budget:
                    i += 1
                    continue
                is_decode = True
            while not self._ensure_blocks(req, req.num_computed_tokens + n):
                victim = self.running.pop()  # newest
                self._preempt(victim)
                out.preempted.append(victim)
                if victim is req:
                    break
            else:
                budget -= n
                samples = is_decode or n >= remaining
                (decodes if is_decode else prefills).append(ScheduledRequest(req, n, is_decode, samples))
                i += 1
                continue
            # req itself was preempted: do not advance i (list shrank)
        # 2) admit waiting requests
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            if self.uses_state and not self.free_state_slots:
                break
            if req.num_computed_tokens == 0 and not req.block_ids:
                cached = self.pool.match_prefix(req.all_token_ids, req.cache_salt)
                if cached:
                    req.block_ids = list(cached)
                    req.num_computed_tokens = len(cached) * self.pool.block_size
            total = req.num_tokens  # preempted requests recompute prompt + generated tokens
            n = total - req.num_computed_tokens
            if self.chunked_prefill:
                n = min(n, budget)
            elif n > budget:
                break
            if not self._ensure_blocks(req, req.num_computed_tokens + n):
                break
            self.waiting.popleft()
            if self.uses_state:
                req.state_slot = self.free_state_slots.pop()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            budget -= n
            samples = req.num_computed_tokens + n >= total
            prefills.append(ScheduledRequest(req, n, False, samples))
        out.scheduled = decodes + prefills
        out.num_tokens = sum(s.num_new_tokens for s in out.scheduled)
        return out

    def finish(self, req: Request) -> None:
        if req in self.running:
            self.running.remove(req)
        self.pool.register_full_blocks(req)
        self.pool.release(req.block_ids)
        req.block_ids = []
        if req.state_slot >= 0:
            self.free_state_slots.append(req.state_slot)
            req.state_slot = -1
        self.finished.append(req)

    def abort(self, request_id: str) -> bool:
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.request_id == request_id:
                    r.status = RequestStatus.FINISHED_ABORTED
                    if q is self.waiting:
                        self.waiting.remove(r)
                    self.finish(r)
                    return True
        return False
