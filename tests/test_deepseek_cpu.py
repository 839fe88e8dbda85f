"""DeepSeek-style MLA + MoE (+ lightning indexer) on the CPU oracle path."""
import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
from vllm_kunlun_b200.config import RopeScaling, deepseek_v3, tiny
from vllm_kunlun_b200.ops.reference import basic as rb


def _cfg(sparse=False, topk=0, fp8=False):
    return tiny(deepseek_v3(fp8=fp8, sparse=sparse), num_layers=3, first_dense_layers=1, vocab_size=320,
                hidden_size=128, num_heads=4, num_kv_heads=4, q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=32,
                qk_rope_head_dim=16, v_head_dim=32, head_dim=48, rotary_dim=16, intermediate_size=256, num_experts=8,
                num_experts_per_tok=2, moe_intermediate_size=128, n_group=4, topk_group=2, max_position=512,
                index_topk=topk, index_n_heads=4 if sparse else 0, index_head_dim=128 if sparse else 0,
                rope_scaling=RopeScaling(type="yarn", factor=4.0, original_max_position=128, mscale=1.0,
                                         mscale_all_dim=1.0), dtype="float32", num_mtp_layers=0)


def _prompts():
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, 320, (n,), generator=g).tolist() for n in (33, 70, 5)]


def test_mla_absorbed_equals_explicit_mha():
    cfg = _cfg()
    llm = LLM(cfg, device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16)
    eng = llm.engine
    attn = eng.runner.model.layers["0"].self_attn
    T = 40
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(T, cfg.hidden_size, generator=g) * 0.5
    req = eng.add_request(list(range(T)), SamplingParams(max_tokens=1))
    sched = eng.scheduler.schedule()
    md, ids, _ = eng.runner.prepare(sched)
    with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
        got = attn(hidden)
        # explicit multi-head attention with materialised K / V
        qkv_a = attn.fused_qkv_a_proj(hidden)
        q_c = attn.q_a_layernorm(qkv_a[:, :64].contiguous())
        kv_c = attn.kv_a_layernorm(qkv_a[:, 64:128].contiguous())
        k_pe = qkv_a[:, 128:]
        q = attn.q_b_proj(q_c).view(T, 4, 48)
        pos = torch.arange(T)
        q_pe = rb.apply_rope(q[..., 32:].reshape(T, -1), pos, attn.cos_sin, 16, False).view(T, 4, 16)
        k_pe = rb.apply_rope(k_pe, pos, attn.cos_sin, 16, False)
        kvb = attn.kv_b_proj.weight.view(4, 64, 64)  # [N, nope+v, rank]
        k_nope = torch.einsum("tr,ndr->tnd", kv_c, kvb[:, :32])
        v = torch.einsum("tr,ndr->tnd", kv_c, kvb[:, 32:])
        s = (torch.einsum("qnd,knd->nqk", q[..., :32], k_nope) + torch.einsum("qnd,kd->nqk", q_pe, k_pe)) * attn.scale
        s = s.masked_fill(~torch.tril(torch.ones(T, T)).bool(), float("-inf"))
        o = torch.einsum("nqk,knd->qnd", s.softmax(-1), v).reshape(T, -1)
        want = attn.o_proj(o)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()


def test_deepseek_engine_chunked_equals_unchunked():
    cfg = _cfg()
    a = LLM(cfg, device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16)
    b = LLM(cfg, device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16,
            max_num_batched_tokens=64)
    with torch.inference_mode():
        b.engine.runner.model.load_state_dict(a.engine.runner.model.state_dict())
        b.engine.runner.model.finish_loading()
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    assert [o.token_ids for o in a.generate(_prompts(), sp)] == [o.token_ids for o in b.generate(_prompts(), sp)]


def test_sparse_with_full_topk_equals_dense():
    dense = LLM(_cfg(), device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16)
    sparse = LLM(_cfg(sparse=True, topk=256), device="cpu", block_size=64, max_model_len=256, max_num_seqs=4,
                 num_gpu_blocks=16)
    with torch.inference_mode():
        sd = dense.engine.runner.model.state_dict()
        missing = sparse.engine.runner.model.load_state_dict(sd, strict=False)
        assert all("indexer" in k for k in missing.missing_keys)
        sparse.engine.runner.model.finish_loading()
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    assert [o.token_ids for o in dense.generate(_prompts(), sp)] == [o.token_ids for o in sparse.generate(_prompts(), sp)]


def test_sparse_small_topk_runs():
    llm = LLM(_cfg(sparse=True, topk=16), device="cpu", block_size=64, max_model_len=256, max_num_seqs=4,
              num_gpu_blocks=16)
    outs = llm.generate(_prompts(), SamplingParams(max_tokens=4, ignore_eos=True))
    assert all(len(o.token_ids) == 4 for o in outs)


def test_sparse_engine_fp8_latent_cache_cpu():
    """``kv_cache_dtype='fp8_ds_mla'`` on the sparse-attention model: 656-byte rows are allocated, written and read
    (oracle kernels on CPU); tokens stay close to the 16-bit cache run."""
    import torch
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import deepseek_v3, tiny
    cfg = tiny(deepseek_v3(fp8=False, sparse=True), num_layers=2, first_dense_layers=1, vocab_size=256, hidden_size=128,
               num_heads=4, num_kv_heads=4, q_lora_rank=64, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=256,
               num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, n_group=1, topk_group=1,
               max_position=512, num_mtp_layers=0, index_topk=16)
    prompts = [torch.randint(0, 256, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (40, 9)]
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    toks = {}
    for kvd in ("auto", "fp8_ds_mla"):
        llm = LLM(cfg, device="cpu", dtype="float32", block_size=64, max_model_len=128, max_num_seqs=2, num_gpu_blocks=8,
                  seed=1, kv_cache_dtype=kvd)
        caches = llm.engine.runner.kv_caches
        first = caches[min(caches)]
        assert (first[0].dtype == torch.uint8) == (kvd == "fp8_ds_mla")
        if kvd == "fp8_ds_mla":
            assert first[0].shape[-1] == 656
        toks[kvd] = [o.token_ids for o in llm.generate(prompts, sp)]
    assert all(len(t) == 4 for t in toks["fp8_ds_mla"])


def _logits_of_steps(llm, prompts, chunk_note=None):
    """Greedy tokens plus the hidden-state fingerprint (first-step logits) of every request."""
    sp = SamplingParams(max_tokens=5, ignore_eos=True, logprobs=None)
    return [o.token_ids for o in llm.generate(prompts, sp)]


@pytest.mark.parametrize("max_batched", [None, 96])
def test_mla_prefill_up_projected_form_equals_absorbed(max_batched):
    """The 192 / 128-style prefill form (new tokens causal + cached context in bounded chunks merged by LSE + the
    other requests of a mixed step on the absorbed form) gives the attention output of the absorbed form."""
    from vllm_kunlun_b200.models.deepseek import MLAAttention
    cfg = _cfg()
    kw = dict(device="cpu", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=32)
    if max_batched:
        kw["max_num_batched_tokens"] = max_batched      # chunked prefill: later chunks see cached context
    a = LLM(cfg, **kw)
    b = LLM(cfg, **kw)
    with torch.inference_mode():
        b.engine.runner.model.load_state_dict(a.engine.runner.model.state_dict())
        b.engine.runner.model.finish_loading()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 320, (n,), generator=g).tolist() for n in (150, 70, 5, 230)]
    calls = {"n": 0, "chunks": 0, "mixed": 0}
    orig = MLAAttention._attend_prefill

    def spy(self, plan, *args):
        calls["n"] += 1
        calls["chunks"] += len(plan["chunks"])
        calls["mixed"] += plan["rest"] is not None
        return orig(self, plan, *args)

    want = _logits_of_steps(a, prompts)
    old = (MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY, MLAAttention.PREFILL_CTX_BYTES,
           MLAAttention._attend_prefill)
    try:
        MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY = True, 16
        MLAAttention.PREFILL_CTX_BYTES = 4 * (32 + 32) * 2 * 64      # 64 context tokens per pass: several chunks
        MLAAttention._attend_prefill = spy
        got = _logits_of_steps(b, prompts)
    finally:
        (MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY, MLAAttention.PREFILL_CTX_BYTES,
         MLAAttention._attend_prefill) = old
    assert calls["n"] > 0
    if max_batched:
        assert calls["chunks"] > calls["n"] // 3 and calls["mixed"] > 0, calls
    assert got == want


def test_mla_prefill_form_attention_rows_match():
    """One attention layer, one step with cached context for one request and none for another: row-level agreement
    of the two forms (not just tokens)."""
    from vllm_kunlun_b200.models.deepseek import MLAAttention
    cfg = _cfg()
    llm = LLM(cfg, device="cpu", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=32,
              max_num_batched_tokens=128)
    eng = llm.engine
    attn = eng.runner.model.layers["0"].self_attn
    eng.add_request(list(range(200)), SamplingParams(max_tokens=1))
    g = torch.Generator().manual_seed(5)
    outs = []
    for step in range(2):       # step 0: 128 new tokens; step 1: 72 new tokens over 128 cached ones
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        hidden = torch.randn(md.num_tokens, cfg.hidden_size, generator=g) * 0.5
        with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
            want = attn(hidden)
            md.extras.pop("mla_prefill_plan", None)
            old = (MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY, MLAAttention.PREFILL_CTX_BYTES)
            try:
                MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY = True, 16
                MLAAttention.PREFILL_CTX_BYTES = 4 * 64 * 2 * 64
                got = attn(hidden)
                plan = md.extras["mla_prefill_plan"]
            finally:
                MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_MIN_QUERY, MLAAttention.PREFILL_CTX_BYTES = old
        assert plan is not None and len(plan["chunks"]) == (2 if step else 0)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (step, (got - want).abs().max())
        outs.append(got)
        # advance the request by hand: the scheduler's bookkeeping for a finished chunk
        for sr in sched.scheduled:
            sr.req.num_computed_tokens += sr.num_new_tokens
