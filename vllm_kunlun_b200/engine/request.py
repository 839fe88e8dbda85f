"""Requests, sampling parameters and outputs of the standalone engine.

The reference owns no engine loop (upstream vLLM's scheduler / KV manager / runner are used,
``vllm_kunlun/platforms/kunlun.py:183-189``); these are this framework's equivalents.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0  # 0 = off
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    ignore_eos: bool = False
    stop_token_ids: tuple = ()
    seed: Optional[int] = None
    logprobs: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


class RequestStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5

    @property
    def finished(self) -> bool:
        return self.value >= 3


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list
    sampling: SamplingParams
    eos_token_id: Optional[int] = None
    arrival_time: float = field(default_factory=time.perf_counter)
    lora_id: int = -1
    mm: Optional[dict] = None  # multimodal: projected image embeddings, prompt rows they replace, M-RoPE positions
    # mutable state
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list = field(default_factory=list)
    num_computed_tokens: int = 0  # tokens whose KV is in the cache
    block_ids: list = field(default_factory=list)
    spec_token_ids: list = field(default_factory=list)  # draft tokens to verify next step
    state_slot: int = -1  # linear-attention state cache slot
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    token_times: list = field(default_factory=list)
    num_pending: int = 0  # tokens launched on the device whose values the host has not seen yet
    num_preemptions: int = 0
    output_logprobs: list = field(default_factory=list)  # log-probability of every sampled token (sampling.logprobs)
    cache_salt: bytes = b""  # prefix-cache hash seed: LoRA adapter id + digest of the multimodal inputs

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def in_prefill(self) -> bool:
        return self.num_computed_tokens < self.num_prompt_tokens

    def append_token(self, tok: int, now: Optional[float] = None, logprob: Optional[float] = None) -> None:
        now = time.perf_counter() if now is None else now
        if self.first_token_time is None:
            self.first_token_time = now
        self.token_times.append(now)
        self.output_token_ids.append(int(tok))
        if logprob is not None:
            self.output_logprobs.append(float(logprob))

    def check_stop(self) -> bool:
        sp = self.sampling
        if self.output_token_ids:
            last = self.output_token_ids[-1]
            if not sp.ignore_eos and self.eos_token_id is not None and last == self.eos_token_id:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
            if last in sp.stop_token_ids:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
        if len(self.output_token_ids) >= sp.max_tokens:
            self.status = RequestStatus.FINISHED_LENGTH
            return True
        return False


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list
    token_ids: list
    finished: bool
    finish_reason: Optional[str] = None
    ttft: Optional[float] = None  # seconds
    tpot: Optional[float] = None  # mean seconds per output token after the first
    text: Optional[str] = None
    logprobs: Optional[list] = None  # per output token, when SamplingParams.logprobs was set

    @classmethod
    def from_request(cls, r: Request) -> "RequestOutput":
        ttft = None if r.first_token_time is None else r.first_token_time - r.arrival_time
        tpot = None
        if len(r.token_times) > 1:
            tpot = (r.token_times[-1] - r.token_times[0]) / (len(r.token_times) - 1)
        reason = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                  RequestStatus.FINISHED_ABORTED: "abort"}.get(r.status)
        return cls(r.request_id, r.prompt_token_ids, list(r.output_token_ids), r.status.finished, reason, ttft, tpot,
                   logprobs=list(r.output_logprobs) if r.sampling.logprobs else None)
