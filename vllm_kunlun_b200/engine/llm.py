"""``LLM``: the user-facing offline entry point (``LLM(...).generate(...)`` as in the reference's
quick start, ``docs/source/quick_start.md:77-106``) and the step loop behind the server.

Every rank of a tensor-/pipeline-parallel job runs the same loop on the same requests (SPMD); the
schedule is a pure function of the request set, and sampled tokens are identical on all ranks
(greedy on all-gathered logits, or a shared seed), so no per-step control messages are needed.
"""
from __future__ import annotations

import itertools
import time
from typing import Iterable, Optional, Sequence, Union

import torch

from ..config import (CacheConfig, CompilationConfig, EngineConfig, LoRAConfig, ModelConfig, ParallelConfig, PRESETS,
                      SchedulerConfig, SpeculativeConfig)
from ..parallel import state as pstate_mod
from .request import Request, RequestOutput, SamplingParams
from .runner import ModelRunner, StepHandle
from .scheduler import BlockPool, Scheduler


def _mm_digest(data: dict) -> bytes:
    """Digest of the pixel data and grid of a request: image placeholder tokens are identical for different images,
    so the prefix-cache hash must see the images themselves."""
    import hashlib
    h = hashlib.blake2b(digest_size=16)
    for key in sorted(data):
        v = data[key]
        h.update(key.encode())
        if isinstance(v, torch.Tensor):
            h.update(str(tuple(v.shape)).encode())
            h.update(v.detach().to("cpu").contiguous().view(torch.uint8).numpy().tobytes())
        else:
            h.update(repr(v.tolist() if hasattr(v, "tolist") else v).encode())
    return h.digest()


class InvalidRequest(ValueError):
    """A request the engine can never serve (the server answers it with HTTP 400)."""


class LLMEngine:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg.finalize()
        if cfg.parallel.world_size > 1 or cfg.parallel.data_parallel_size > 1:
            pstate_mod.init_distributed()
        self.pstate = pstate_mod.initialize_model_parallel(
            tp=cfg.parallel.tensor_parallel_size, pp=cfg.parallel.pipeline_parallel_size,
            dp=cfg.parallel.data_parallel_size, ep=cfg.parallel.enable_expert_parallel,
            dcp=cfg.parallel.decode_context_parallel_size, device=cfg.device,
            fused_collectives=cfg.parallel.fused_collectives) \
            if torch.distributed.is_initialized() else pstate_mod.get_state()
        self.runner = ModelRunner(self.cfg, self.pstate)
        # with decode context parallelism a block spans block_size tokens on EACH rank of the DCP group
        self.pool = BlockPool(self.runner.num_blocks, self.runner.tokens_per_block, self.cfg.cache.enable_prefix_caching)
        self.scheduler = Scheduler(
            self.pool, self.cfg.scheduler.max_num_seqs, self.cfg.scheduler.max_num_batched_tokens,
            self.cfg.scheduler.max_model_len, self.cfg.scheduler.enable_chunked_prefill,
            self.cfg.speculative.num_speculative_tokens, getattr(self.runner, "num_state_slots", 0))
        self.spec = None
        if self.cfg.speculative.method:
            from .spec_decode import build_proposer
            self.spec = build_proposer(self)
        # async scheduling: launch step i+1 before reading step i's tokens (not with speculation,
        # whose accepted length decides the next step's inputs)
        self.async_scheduling = self.runner.is_cuda and self.spec is None
        self._inflight: Optional[StepHandle] = None
        self._ids = itertools.count()
        # host-side failure detection between steps (parallel/health.py): every N-th step the ranks shake hands
        # through the job's key-value store before launching; off unless B200_HEALTH_CHECK_INTERVAL > 0
        self.monitor = None
        from .. import envs
        self._health_every = int(envs.B200_HEALTH_CHECK_INTERVAL)
        if self._health_every > 0:
            from ..parallel.health import RankMonitor
            self.monitor = RankMonitor.from_default_group(timeout=float(envs.B200_HEALTH_TIMEOUT_S))
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0,
                      "spec_proposed": 0, "spec_accepted": 0}

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_token_ids: Sequence[int], sampling: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, eos_token_id: Optional[int] = None, lora_id: int = -1,
                    multi_modal_data: Optional[dict] = None):
        """``multi_modal_data``: ``{"pixel_values": tensor, "image_grid_thw": [[t, h, w], ...]}`` for
        vision-language models; the vision tower runs here, once per request."""
        rid = request_id or f"req-{next(self._ids)}"
        sampling = sampling or SamplingParams()
        self.validate_request(prompt_token_ids, sampling)
        req = Request(rid, list(prompt_token_ids), sampling, eos_token_id, lora_id=lora_id)
        salt = b"" if lora_id < 0 else f"lora{lora_id}".encode()
        if multi_modal_data is not None:
            req.mm = self.runner.encode_multimodal(req.prompt_token_ids, multi_modal_data)
            if self.cfg.cache.enable_prefix_caching:
                salt += b"|mm" + _mm_digest(multi_modal_data)
        req.cache_salt = salt
        self.scheduler.add(req)
        return req

    def validate_request(self, prompt_token_ids: Sequence[int], sampling: SamplingParams) -> None:
        """Raise :class:`InvalidRequest` for a request that could never be scheduled or sampled: an empty prompt, a
        prompt that leaves no room for one generated token, a prompt larger than the whole block pool, token ids
        outside the vocabulary, sampling parameters outside their domains (upstream answers these with HTTP 400)."""
        n = len(prompt_token_ids)
        mml = self.cfg.scheduler.max_model_len
        if n == 0:
            raise InvalidRequest("the prompt is empty")
        if n >= mml:
            raise InvalidRequest(f"the prompt has {n} tokens; with max_model_len={mml} there is no room to generate")
        need = -(-(n + 1) // self.pool.block_size)
        if need > self.pool.num_blocks:
            raise InvalidRequest(f"the prompt needs {need} KV blocks but the pool has {self.pool.num_blocks}")
        V = self.cfg.model.vocab_size
        lo, hi = min(prompt_token_ids), max(prompt_token_ids)
        if lo < 0 or hi >= V:
            raise InvalidRequest(f"token id {lo if lo < 0 else hi} is outside the vocabulary [0, {V})")
        sp = sampling
        if sp.max_tokens < 1:
            raise InvalidRequest("max_tokens must be at least 1")
        if sp.temperature < 0 or sp.temperature != sp.temperature:
            raise InvalidRequest("temperature must be non-negative")
        if not (0.0 < sp.top_p <= 1.0):
            raise InvalidRequest("top_p must be in (0, 1]")
        if sp.top_k < 0:
            raise InvalidRequest("top_k must be non-negative (0 disables it)")
        if not sp.repetition_penalty > 0:
            raise InvalidRequest("repetition_penalty must be positive")

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id)

    def abort_all(self) -> list:
        """Drop every request (after a failed step): frees their blocks; returns the dropped requests."""
        self._inflight = None
        dropped = list(self.scheduler.running) + list(self.scheduler.waiting)
        for r in dropped:
            self.scheduler.abort(r.request_id)
        return dropped

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------ stepping
    def _process(self, h: StepHandle) -> list:
        """Append sampled tokens, run stop checks, free finished requests."""
        toks = h.wait().tolist()
        lps = None if h.logprobs_cpu is None else h.logprobs_cpu.tolist()
        now = time.perf_counter()
        finished = []
        row = 0
        for req, rows in zip(h.sample_reqs, h.rows_per_req):
            vals = toks[row:row + rows]
            lp = None if lps is None or not req.sampling.logprobs else lps[row:row + rows]
            row += rows
            req.num_pending = max(0, req.num_pending - 1)
            if req.status.finished:
                continue  # finished while this step was in flight: drop the extra token
            if self.spec is not None and rows > 1:
                vals = self.spec.accept(req, vals, self.stats)
            for j, v in enumerate(vals):
                req.append_token(v, now, None if lp is None or j >= len(lp) else lp[j])
                if req.check_stop():
                    self.scheduler.finish(req)
                    finished.append(req)
                    break
        return finished

    def step(self) -> list:
        """Run one engine iteration; returns requests that finished."""
        if self._inflight is not None and self._needs_host_tokens():
            # repetition penalties and per-request seeds read the full token history on the host: finish the step in
            # flight before the next one is prepared
            done = self._process(self._inflight)
            self._inflight = None
            return done + self.step() if self.scheduler.has_work() else done
        sched = self.scheduler.schedule()
        self.stats["preemptions"] += len(sched.preempted)
        finished = []
        if sched.empty:
            if self._inflight is not None:
                finished = self._process(self._inflight)
                self._inflight = None
            return finished
        if self.monitor is not None and self.stats["steps"] % self._health_every == 0:
            # no kernel of the coming step has been launched yet: a peer that left or stopped beating surfaces
            # here as RankLeft / RankTimeout instead of as a collective that never completes
            self.monitor.check(wait_for_step=self.monitor.beat())
        h = self.runner.execute(sched)
        self.stats["steps"] += 1
        for sr in sched.scheduled:
            self.stats["decode_tokens" if sr.is_decode else "prefill_tokens"] += sr.num_new_tokens
            if sr.samples:
                sr.req.num_pending += 1
        if self.async_scheduling:
            prev, self._inflight = self._inflight, h
            if prev is not None:
                finished = self._process(prev)
            # a request that will hit max_tokens with its pending token must not be scheduled again
            for sr in sched.scheduled:
                r = sr.req
                if sr.samples and len(r.output_token_ids) + r.num_pending >= r.sampling.max_tokens:
                    self._drain()
                    finished += self._finished_since
                    break
        else:
            finished = self._process(h)
            if self.spec is not None:
                self.spec.propose(h, self.stats)
        return finished

    _finished_since: list = []

    def _needs_host_tokens(self) -> bool:
        return any(r.sampling.repetition_penalty != 1.0 or (r.sampling.seed is not None and not r.sampling.greedy)
                   for r in self.scheduler.running)

    def _drain(self):
        self._finished_since = []
        if self._inflight is not None:
            self._finished_since = self._process(self._inflight)
            self._inflight = None

    def run_until_done(self) -> list:
        done = []
        while self.has_unfinished():
            done += self.step()
        return done


class LLM:
    """Offline inference front-end.

    ``model`` is a preset name (random-init weights of that architecture), a :class:`ModelConfig`,
    or a directory with ``config.json`` + safetensors (the checkpoint format the reference loads,
    including fp8 block-128 ``weight_scale_inv`` tensors)."""

    def __init__(self, model: Union[str, ModelConfig], tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                 enable_expert_parallel: bool = False, device: Optional[str] = None, dtype: Optional[str] = None,
                 block_size: int = 16, max_model_len: int = 8192, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, gpu_memory_utilization: float = 0.9,
                 num_gpu_blocks: Optional[int] = None, enable_prefix_caching: bool = False,
                 enforce_eager: bool = False, speculative_config: Optional[dict] = None, seed: int = 0,
                 enable_chunked_prefill: bool = True, kv_cache_dtype: str = "auto",
                 fused_collectives: bool = True, tokenizer=None, enable_lora: bool = False, max_loras: int = 4,
                 max_lora_rank: int = 16, decode_context_parallel_size: int = 1, data_parallel_size: int = 1):
        """``data_parallel_size`` > 1: the job's ranks form that many independent replicas of ``tensor_parallel_size x
        pipeline_parallel_size`` ranks; every replica schedules and serves its own requests (the caller gives each
        replica its share, ``engine.pstate.dp_rank`` tells which replica a rank belongs to)."""
        import os
        weights = None
        if isinstance(model, ModelConfig):
            mc = model
        elif model in PRESETS:
            mc = PRESETS[model]()
        elif os.path.isdir(model):
            mc = ModelConfig.from_pretrained(model)
            weights = model
        else:
            raise ValueError(f"unknown model {model!r}")
        if dtype:
            mc.dtype = dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        if device == "cuda":
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
            torch.cuda.set_device(device)
        spec = SpeculativeConfig(**(speculative_config or {}))
        cfg = EngineConfig(
            model=mc,
            cache=CacheConfig(block_size=block_size, num_blocks=num_gpu_blocks,
                              gpu_memory_utilization=gpu_memory_utilization, cache_dtype=kv_cache_dtype,
                              enable_prefix_caching=enable_prefix_caching),
            parallel=ParallelConfig(tensor_parallel_size, pipeline_parallel_size, data_parallel_size,
                                    enable_expert_parallel=enable_expert_parallel,
                                    decode_context_parallel_size=decode_context_parallel_size,
                                    fused_collectives=fused_collectives),
            scheduler=SchedulerConfig(max_num_seqs, max_num_batched_tokens, max_model_len, enable_chunked_prefill),
            speculative=spec,
            compilation=CompilationConfig(mode="none" if enforce_eager else "full_decode"),
            lora=LoRAConfig(enable_lora, max_loras, max_lora_rank),
            device=device, seed=seed, weights_path=weights)
        self.engine = LLMEngine(cfg)
        self.tokenizer = tokenizer
        self.eos_token_id = getattr(tokenizer, "eos_token_id", None)

    def add_lora(self, lora_request) -> int:
        """Load an adapter (:class:`vllm_kunlun_b200.lora.LoRARequest`) into a slot; returns the slot."""
        assert self.engine.runner.lora is not None, "construct the LLM with enable_lora=True"
        with torch.inference_mode():
            return self.engine.runner.lora.add_adapter(lora_request)

    def generate(self, prompt_token_ids: Iterable[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 lora_request=None, multi_modal_data=None) -> list:
        prompts = list(prompt_token_ids)
        if multi_modal_data is None or isinstance(multi_modal_data, dict):
            multi_modal_data = [multi_modal_data] * len(prompts)
        if lora_request is None or not isinstance(lora_request, (list, tuple)):
            lora_request = [lora_request] * len(prompts)
        for lr in lora_request:
            if lr is not None:
                self.add_lora(lr)
        if isinstance(prompts[0], str):
            assert self.tokenizer is not None, "string prompts need a tokenizer"
            prompts = [self.tokenizer.encode(p) for p in prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        import copy
        reqs = [self.engine.add_request(p, copy.copy(sp), eos_token_id=self.eos_token_id,
                                        lora_id=-1 if lr is None else lr.lora_int_id, multi_modal_data=mm)
                for p, sp, lr, mm in zip(prompts, sampling_params, lora_request, multi_modal_data)]
        self.engine.run_until_done()
        outs = [RequestOutput.from_request(r) for r in reqs]
        if self.tokenizer is not None:
            for o in outs:
                o.text = self.tokenizer.decode(o.token_ids)
        return outs
