"""Request validation, failure handling and cache-salting on the CPU engine: a bad request fails alone, a failed
step fails its requests but not the server, a device status word surfaces as a step error."""
import json
import math

import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import qwen2_0_5b, tiny
from vllm_kunlun_b200.engine.llm import InvalidRequest
from vllm_kunlun_b200.engine.runner import DeviceWaitTimeout, StepHandle
from vllm_kunlun_b200.engine.scheduler import BlockPool


def _llm(**kw):
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=512, dtype="float32")
    base = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    base.update(kw)
    return LLM(cfg, **base)


def test_unservable_requests_are_rejected_and_the_engine_keeps_working():
    llm = _llm()
    eng = llm.engine
    with pytest.raises(InvalidRequest, match="empty"):
        eng.add_request([], SamplingParams(max_tokens=4))
    with pytest.raises(InvalidRequest, match="no room"):
        eng.add_request([1] * 200, SamplingParams(max_tokens=4))       # longer than max_model_len
    with pytest.raises(InvalidRequest, match="no room"):
        eng.add_request([1] * 128, SamplingParams(max_tokens=4))       # exactly max_model_len
    with pytest.raises(InvalidRequest, match="vocabulary"):
        eng.add_request([1, 2, 500], SamplingParams(max_tokens=4))
    for bad in (dict(max_tokens=0), dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-2),
                dict(repetition_penalty=0.0)):
        with pytest.raises(InvalidRequest):
            eng.add_request([1, 2, 3], SamplingParams(**bad))
    small = _llm(num_gpu_blocks=2, max_model_len=128)
    with pytest.raises(InvalidRequest, match="KV blocks"):
        small.engine.add_request([1] * 100, SamplingParams(max_tokens=4))
    # nothing was queued, the pool is untouched and a good request still runs
    assert not eng.has_unfinished() and eng.pool.num_free == 32
    out = llm.generate([[5, 6, 7]], SamplingParams(max_tokens=4, ignore_eos=True))[0]
    assert len(out.token_ids) == 4
    # a prompt of max_model_len - 1 tokens is the longest servable one: exactly one token comes out
    out = llm.generate([[3] * 127], SamplingParams(max_tokens=9, ignore_eos=True))[0]
    assert len(out.token_ids) == 1 and out.finish_reason == "length"


def test_speculative_drafts_stop_at_max_model_len():
    """Verify steps near the length limit must not index past the block table (drafts are cut to the room left)."""
    llm = _llm(speculative_config={"method": "ngram", "num_speculative_tokens": 3}, max_model_len=64)
    prompt = [7, 8, 9, 10] * 14  # 56 tokens, repetitive: the n-gram proposer always finds drafts
    out = llm.generate([prompt], SamplingParams(max_tokens=64, ignore_eos=True))[0]
    assert len(prompt) + len(out.token_ids) == 64
    ref = _llm(max_model_len=64).generate([prompt], SamplingParams(max_tokens=64, ignore_eos=True))[0]
    assert out.token_ids == ref.token_ids


def test_repetition_penalty_seed_and_logprobs_reach_the_sampler():
    llm = _llm()
    p = [5, 6, 7, 8]
    plain = llm.generate([p], SamplingParams(max_tokens=12, ignore_eos=True))[0]
    pen = llm.generate([p], SamplingParams(max_tokens=12, ignore_eos=True, repetition_penalty=1e4))[0]
    # an extreme penalty forbids every token seen so far (greedy): no token repeats, none comes from the prompt
    assert len(set(pen.token_ids)) == len(pen.token_ids) and not set(pen.token_ids) & set(p)
    assert pen.token_ids != plain.token_ids or len(set(plain.token_ids)) == len(plain.token_ids)
    # a per-request seed reproduces its tokens whatever else shares the batch
    sp = SamplingParams(max_tokens=10, ignore_eos=True, temperature=2.0, seed=1234)
    alone = llm.generate([p], sp)[0].token_ids
    mixed = llm.generate([[9, 9, 9], p, [1, 2]], [SamplingParams(max_tokens=7, temperature=1.0, ignore_eos=True), sp,
                                                   SamplingParams(max_tokens=3, ignore_eos=True)])[1].token_ids
    assert alone == mixed
    other = llm.generate([p], SamplingParams(max_tokens=10, ignore_eos=True, temperature=2.0, seed=99))[0].token_ids
    assert other != alone
    # log-probabilities of the sampled tokens: greedy tokens carry the row maximum
    lp = llm.generate([p], SamplingParams(max_tokens=5, ignore_eos=True, logprobs=True))[0]
    assert lp.token_ids == plain.token_ids[:5] and len(lp.logprobs) == 5
    assert all(-math.log(128) - 1e-3 <= v <= 0.0 for v in lp.logprobs)


def test_prefix_cache_is_salted_by_adapter_and_image():
    pool = BlockPool(16, 4, enable_prefix_caching=True)
    from vllm_kunlun_b200.engine.request import Request
    toks = list(range(13))

    def finished(salt):
        r = Request("r" + salt.decode(), list(toks), SamplingParams())
        r.cache_salt = salt
        r.block_ids = pool.allocate(4)
        r.num_computed_tokens = 13
        pool.register_full_blocks(r)
        pool.release(r.block_ids)
        return r
    finished(b"lora1")
    assert len(pool.match_prefix(toks, b"lora1")) == 3
    assert pool.match_prefix(toks, b"lora2") == []     # another adapter: same tokens, different KV
    assert pool.match_prefix(toks, b"") == []          # the base model neither
    from vllm_kunlun_b200.engine.llm import _mm_digest
    a = {"pixel_values": torch.zeros(4, 6), "image_grid_thw": [[1, 2, 2]]}
    b = {"pixel_values": torch.ones(4, 6), "image_grid_thw": [[1, 2, 2]]}
    assert _mm_digest(a) != _mm_digest(b) and _mm_digest(a) == _mm_digest(dict(a))


def test_engine_prefix_cache_keeps_adapters_apart():
    llm = _llm(enable_prefix_caching=True, max_model_len=256)
    eng = llm.engine
    shared = list(range(5, 5 + 70))
    sp = SamplingParams(max_tokens=2, ignore_eos=True)
    eng.add_request(shared, sp, lora_id=-1)
    eng.run_until_done()
    before = eng.stats["prefill_tokens"]
    r = eng.add_request(shared, sp, lora_id=-1)
    eng.run_until_done()
    assert eng.stats["prefill_tokens"] - before < len(shared)  # base model again: the prefix is reused
    before = eng.stats["prefill_tokens"]
    r = eng.add_request(shared, sp, lora_id=3)
    assert r.cache_salt == b"lora3"
    eng.run_until_done()
    assert eng.stats["prefill_tokens"] - before == len(shared)  # an adapter: nothing is reused


def test_status_word_turns_into_a_step_error():
    """The device status words travel with the tokens; a non-zero word fails the step that produced it."""
    ok = StepHandle(None, [], [], torch.zeros(1), torch.tensor([7]), None, status_cpu=torch.tensor([0, 0]),
                    status_names=("tp_peer", "gemm"))
    assert ok.wait().tolist() == [7]
    bad = StepHandle(None, [], [], torch.zeros(1), torch.tensor([7]), None, status_cpu=torch.tensor([0, 211]),
                     status_names=("tp_peer", "gemm"))
    with pytest.raises(DeviceWaitTimeout, match="gemm=211"):
        bad.wait()


def test_server_answers_400_and_survives_a_failed_step():
    from fastapi.testclient import TestClient

    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    llm = _llm()
    app = build_app(llm, "tiny")
    eng = llm.engine
    with TestClient(app) as c:
        good = {"prompt": [5, 6, 7, 8], "max_tokens": 3, "temperature": 0, "ignore_eos": True}
        r = c.post("/v1/completions", json={"prompt": [1] * 300, "max_tokens": 4})
        assert r.status_code == 400 and "no room" in r.json()["error"]["message"]
        assert c.post("/v1/completions", json={"prompt": [], "max_tokens": 4}).status_code == 400
        assert c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 0}).status_code == 400
        assert c.post("/v1/completions", json={"prompt": [1, 2], "top_p": "x"}).status_code == 400
        assert c.post("/v1/completions", json=good).status_code == 200
        # one step blows up: the request in flight gets a 500, the loop goes on and later requests are served
        real_step, state = eng.step, {"n": 0}

        def flaky():
            state["n"] += 1
            if state["n"] == 1:
                raise RuntimeError("injected step failure")
            return real_step()
        eng.step = flaky
        r = c.post("/v1/completions", json=good)
        assert r.status_code == 500 and "injected" in r.json()["error"]["message"]
        assert eng.pool.num_free == 32 and not eng.has_unfinished()
        r = c.post("/v1/completions", json=good)
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 3
        assert c.get("/health").status_code == 200
        # a device-side time-out marks the server unhealthy (caches may hold wrong data) but it still answers
        state["n"] = -10**9

        def timeout_once():
            eng.step = real_step
            raise DeviceWaitTimeout("tp_peer=211")
        eng.step = timeout_once
        assert c.post("/v1/completions", json=good).status_code == 500
        assert c.get("/health").status_code == 503
        assert c.post("/v1/completions", json=good).status_code == 200
        assert "b200_requests_total" in c.get("/metrics").text
