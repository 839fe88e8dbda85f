"""End-to-end plumbing on CPU: paged-KV engine vs a plain full-context PyTorch forward."""
import dataclasses

import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import qwen2_0_5b
from vllm_kunlun_b200.ops.reference import basic as rb


def plain_forward(model, cfg, ids):
    """HF-style full-context forward in fp32 (no KV cache, no paging)."""
    T = len(ids)
    x = model.embed_tokens.weight[torch.tensor(ids)].float()
    pos = torch.arange(T)
    cs = rb.build_cos_sin_cache(cfg.head_dim, cfg.max_position if cfg.max_position < 4096 else 4096,
                                cfg.rope_theta, None)
    g = cfg.num_heads // cfg.num_kv_heads
    for i in range(cfg.num_layers):
        L = model.layers[str(i)]
        h = rb.rmsnorm(x, L.input_layernorm.weight, cfg.rms_norm_eps)
        qkv = h @ L.self_attn.qkv_proj.weight.float().T
        if L.self_attn.qkv_proj.bias is not None:
            qkv = qkv + L.self_attn.qkv_proj.bias.float()
        q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], -1)
        if cfg.qk_norm:
            q = rb.rmsnorm(q.reshape(T, -1, cfg.head_dim), L.self_attn.q_norm.weight, cfg.rms_norm_eps).reshape(T, -1)
            k = rb.rmsnorm(k.reshape(T, -1, cfg.head_dim), L.self_attn.k_norm.weight, cfg.rms_norm_eps).reshape(T, -1)
        q = rb.apply_rope(q, pos, cs, cfg.head_dim, True).reshape(T, cfg.num_heads, cfg.head_dim)
        k = rb.apply_rope(k, pos, cs, cfg.head_dim, True).reshape(T, cfg.num_kv_heads, cfg.head_dim)
        v = v.reshape(T, cfg.num_kv_heads, cfg.head_dim)
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * cfg.head_dim ** -0.5
        s = s.masked_fill(~torch.tril(torch.ones(T, T)).bool(), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, -1)
        x = x + o @ L.self_attn.o_proj.weight.float().T
        h = rb.rmsnorm(x, L.post_attention_layernorm.weight, cfg.rms_norm_eps)
        gu = h @ L.mlp.gate_up_proj.weight.float().T
        x = x + rb.silu_and_mul(gu) @ L.mlp.down_proj.weight.float().T
    x = rb.rmsnorm(x, model.norm.weight, cfg.rms_norm_eps)
    return x @ model.lm_head.weight.float().T


def greedy_plain(model, cfg, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain_forward(model, cfg, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("chunk", [8192, 48])
def test_small_dense_matches_plain(chunk):
    cfg = dataclasses.replace(qwen2_0_5b(), num_layers=3, vocab_size=1000, max_position=4096)
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=256, max_num_seqs=8,
              max_num_batched_tokens=chunk, num_gpu_blocks=128)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (37, 16, 65, 5)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    model = llm.engine.runner.model
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_plain(model, cfg, p, 6)
        assert o.finish_reason == "length"


def test_preemption_recompute():
    cfg = dataclasses.replace(qwen2_0_5b(), num_layers=2, vocab_size=500, max_position=4096)
    # pool too small for all sequences at once -> some are preempted and recomputed
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=256, num_gpu_blocks=9)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 500, (40,), generator=g).tolist() for _ in range(3)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))
    model = llm.engine.runner.model
    assert llm.engine.stats["preemptions"] > 0
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_plain(model, cfg, p, 20)


def test_profile_run_leaves_engine_usable():
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    want = llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=4, ignore_eos=True))[0].token_ids
    assert llm.engine.runner.profile_run(64) == 0
    assert llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=4, ignore_eos=True))[0].token_ids == want


def _tiny_llm(**kw):
    from vllm_kunlun_b200.config import tiny
    cfg = tiny(qwen2_0_5b(), num_layers=2, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=512, dtype="float32")
    base = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64)
    base.update(kw)
    return LLM(cfg, **base)


def test_prefix_caching_reuses_blocks_and_keeps_outputs():
    shared = list(range(5, 5 + 70))  # four full blocks and a bit
    prompts = [shared + [100, 101], shared + [102], shared + [100, 101]]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    plain = [o.token_ids for o in _tiny_llm().generate(prompts, sp)]
    llm = _tiny_llm(enable_prefix_caching=True)
    first = llm.generate(prompts[:1], sp)[0].token_ids
    before = llm.engine.stats["prefill_tokens"]
    rest = [o.token_ids for o in llm.generate(prompts[1:], sp)]
    assert [first] + rest == plain
    # the two later prompts recompute only what lies beyond the cached 64-token prefix
    assert llm.engine.stats["prefill_tokens"] - before <= 2 * (len(shared) + 2 - 64)


def test_abort_frees_blocks_and_other_requests_finish():
    llm = _tiny_llm()
    eng = llm.engine
    free0 = eng.pool.num_free
    a = eng.add_request(list(range(3, 40)), SamplingParams(max_tokens=50, ignore_eos=True))
    b = eng.add_request(list(range(50, 70)), SamplingParams(max_tokens=6, ignore_eos=True))
    for _ in range(3):
        eng.step()
    assert eng.abort(a.request_id)
    eng.run_until_done()
    assert b.status.finished and len(b.output_token_ids) == 6
    assert a.status.name == "FINISHED_ABORTED" and len(a.output_token_ids) < 50
    assert eng.pool.num_free == free0


def test_stop_tokens_eos_and_sampling_parameters():
    llm = _tiny_llm()
    greedy = llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids
    stop_at = greedy[2]
    cut = llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=8, stop_token_ids=(stop_at,)))[0]
    assert cut.token_ids[-1] == stop_at and len(cut.token_ids) <= 3 and cut.finish_reason == "stop"
    # top_k = 1 is greedy whatever the temperature; different seeds at high temperature give different text
    k1 = llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=8, temperature=1.5, top_k=1, ignore_eos=True))[0].token_ids
    assert k1 == greedy
    hot = [_tiny_llm(seed=s).generate([[5, 6, 7, 8]], SamplingParams(max_tokens=12, temperature=5.0, ignore_eos=True))[0].token_ids
           for s in (0, 0, 1)]
    assert hot[0] == hot[1]
