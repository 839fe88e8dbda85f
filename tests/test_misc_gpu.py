"""Sampling, gated-delta-net, conv, LoRA and MTP-glue kernels against their fp32 oracles."""
import pytest
import torch

from vllm_kunlun_b200 import ops
from vllm_kunlun_b200.ops.reference import basic as rb
from vllm_kunlun_b200.ops.reference import misc as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _surviving(logits, temperature, top_k, top_p):
    lg = logits.float() / temperature.unsqueeze(1)
    V = lg.shape[1]
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k)
    return ref.apply_top_k_top_p(lg.cpu(), k.cpu(), top_p.cpu()).softmax(-1)


@pytest.mark.parametrize("V", [1000, 151936])
def test_topk_topp_sample_matches_sort_based_masking(V):
    torch.manual_seed(0)
    B = 12
    logits = (torch.randn(B, V, device=DEV) * 3).to(torch.bfloat16)
    temp = torch.tensor([0.0, 1.0, 0.7, 1.3] * 3, device=DEV)
    top_k = torch.tensor([0, 0, 50, 5, 0, 1, 20, 0, 7, 0, 0, 100], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5, 0.2, 1.0, 0.8, 1.0, 0.95, 0.05, 1.0, 0.6], device=DEV)
    noise = torch.empty(B, V, device=DEV).exponential_()
    got = ops.topk_topp_sample(logits, temp, top_k, top_p, noise=noise).cpu()
    t_safe = torch.where(temp == 0, torch.ones_like(temp), temp)
    probs = _surviving(logits, t_safe, top_k, top_p)
    want = (probs / noise.cpu()).argmax(-1)
    greedy = logits.float().argmax(-1).cpu()
    for b in range(B):
        if temp[b] == 0:
            assert got[b] == greedy[b]
        else:
            # the drawn token must be in the reference's surviving set; away from threshold ties it is the same token
            assert probs[b, got[b]] > 0, b
    same = (got == torch.where(temp.cpu() == 0, greedy, want)).float().mean()
    assert same >= 0.9
    # in-kernel generator: draws differ between calls and stay inside the surviving set
    a = ops.topk_topp_sample(logits, temp, top_k, top_p, seed=1).cpu()
    b2 = ops.topk_topp_sample(logits, temp, top_k, top_p, seed=1).cpu()
    for b in range(B):
        assert probs[b, a[b]] > 0 or temp[b] == 0
    assert (a != b2).any()


def test_sampling_distribution_is_unbiased():
    torch.manual_seed(1)
    V, n = 8, 4096
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -0.5, -1.0, -2.0, -3.0], device=DEV)
    logits = row.repeat(n, 1)
    temp = torch.ones(n, device=DEV)
    draws = ops.topk_topp_sample(logits, temp, None, None, seed=7).cpu()
    freq = torch.bincount(draws, minlength=V).float() / n
    torch.testing.assert_close(freq, row.softmax(-1).cpu(), atol=0.03, rtol=0)


def test_repetition_penalty():
    torch.manual_seed(2)
    B, V = 4, 5000
    logits = torch.randn(B, V, device=DEV)
    toks = torch.randint(0, V, (B, 64), device=DEV)
    toks[:, 10] = toks[:, 3]  # duplicates are penalised once
    n = torch.tensor([64, 10, 0, 33], dtype=torch.int32, device=DEV)
    pen = torch.tensor([1.2, 2.0, 1.5, 1.0], device=DEV)
    want = ops.apply_repetition_penalty(logits.cpu().clone(), toks.cpu(), n.cpu(), pen.cpu())
    got = ops.apply_repetition_penalty(logits.clone(), toks, n, pen)
    torch.testing.assert_close(got.cpu(), want)


def test_rejection_sample_kernel_matches_vectorised_reference():
    from vllm_kunlun_b200.sample.rejection_sampler import RejectionSampler
    torch.manual_seed(3)
    B, S, V = 6, 3, 2000
    num_draft = torch.tensor([3, 2, 0, 3, 1, 3], device=DEV)
    n = int(num_draft.sum())
    tp = torch.randn(n, V, device=DEV).softmax(-1)
    dp = torch.randn(n, V, device=DEV).softmax(-1)
    draft = tp.argmax(-1).clone()
    draft[1] = (draft[1] + 1) % V
    draft[4] = (draft[4] + 5) % V
    bonus = torch.randint(0, V, (B,), device=DEV)
    greedy = torch.tensor([True, False, True, False, True, False], device=DEV)
    u = torch.rand(n, device=DEV)
    rq = torch.empty(B, V, device=DEV).exponential_()
    for draft_probs in (dp, None):
        want = RejectionSampler().forward(draft, num_draft, tp, bonus, greedy, draft_probs, u, rq, S)
        got = ops.rejection_sample(draft, num_draft, tp, bonus, greedy, draft_probs, u, rq, S)
        assert torch.equal(got.cpu(), want.cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_causal_conv1d_fn_and_update(dtype):
    torch.manual_seed(4)
    C, W, slots = 384, 4, 6
    cu = torch.tensor([0, 7, 7, 9, 40], dtype=torch.int32)
    T = int(cu[-1])
    x_wide = torch.randn(T, C + 64).to(dtype)
    x = x_wide[:, :C]  # a column slice of a wider projection
    w = (torch.randn(C, W) * 0.5).to(dtype)
    bias = torch.randn(C).to(dtype)
    states = torch.randn(slots, W - 1, C).to(dtype)
    idx = torch.tensor([3, 0, 5, 1], dtype=torch.int32)
    init = torch.tensor([1, 0, 0, 1], dtype=torch.int32)
    s_ref = states.clone()
    want = ref.causal_conv1d_fn(x, w, bias, cu, s_ref, idx, init, True)
    s_dev = states.to(DEV)
    got = ops.causal_conv1d_fn(x_wide.to(DEV)[:, :C], w.to(DEV), bias.to(DEV), cu.to(DEV), s_dev, idx.to(DEV), init.to(DEV), True)
    tol = dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol)
    torch.testing.assert_close(s_dev.cpu().float(), s_ref.float(), **tol)
    # decode step
    xb = torch.randn(4, C).to(dtype)
    idx2 = torch.tensor([3, -1, 5, 1], dtype=torch.int32)
    want2 = ref.causal_conv1d_update(xb, s_ref, w, bias, idx2, True)
    got2 = ops.causal_conv1d_update(xb.to(DEV), s_dev, w.to(DEV), bias.to(DEV), idx2.to(DEV), True)
    torch.testing.assert_close(got2.cpu().float(), want2.float(), **tol)
    torch.testing.assert_close(s_dev.cpu().float(), s_ref.float(), **tol)


@pytest.mark.parametrize("Dk,Dv,Hk,Hv", [(128, 128, 2, 4), (64, 32, 2, 2)])
def test_gated_delta_rule_varlen(Dk, Dv, Hk, Hv):
    torch.manual_seed(5)
    cu = torch.tensor([0, 1, 50, 50, 180], dtype=torch.int32)
    T = int(cu[-1])
    C = 2 * Hk * Dk + Hv * Dv
    mixed = torch.randn(T, C).to(torch.bfloat16)
    q = mixed[:, : Hk * Dk].view(T, Hk, Dk)
    k = mixed[:, Hk * Dk:2 * Hk * Dk].view(T, Hk, Dk)
    v = mixed[:, 2 * Hk * Dk:].view(T, Hv, Dv)
    A_log, dt_bias = torch.rand(Hv), torch.rand(Hv)
    a, b = torch.randn(T, Hv).to(torch.bfloat16), torch.randn(T, Hv).to(torch.bfloat16)
    g_ref, beta_ref = ops.fused_gdn_gating(A_log, a, b, dt_bias)
    g, beta = ops.fused_gdn_gating(A_log.to(DEV), a.to(DEV), b.to(DEV), dt_bias.to(DEV))
    torch.testing.assert_close(g.cpu(), g_ref, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(beta.cpu(), beta_ref, atol=1e-5, rtol=1e-5)
    states = torch.randn(5, Hv, Dv, Dk) * 0.1
    idx = torch.tensor([2, 0, 4, 1], dtype=torch.int32)
    init = torch.tensor([1, 1, 0, 0], dtype=torch.int32)
    s_ref = states.clone()
    want = ops.gated_delta_rule(q, k, v, g_ref, beta_ref, s_ref, cu, idx, init)
    s_dev = states.to(DEV)
    md = mixed.to(DEV)
    got = ops.gated_delta_rule(md[:, : Hk * Dk].view(T, Hk, Dk), md[:, Hk * Dk:2 * Hk * Dk].view(T, Hk, Dk),
                               md[:, 2 * Hk * Dk:].view(T, Hv, Dv), g, beta, s_dev, cu.to(DEV), idx.to(DEV), init.to(DEV))
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(s_dev.cpu(), s_ref, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pattern", ["random", "segments"])
@pytest.mark.parametrize("N,offset,r", [(640, 128, 16), (333, 5, 8), (1030, 0, 12)])
def test_lora_shrink_expand(dtype, pattern, N, offset, r):
    """Token-tiled shrink / expand kernels vs the oracle: tiles whose tokens share an adapter (prefill segments), tiles
    with several adapters and base-model rows (-1), whole tiles of base-model rows, a token count off the tile sizes,
    odd column counts / offsets (no paired 4-byte stores), ranks that are not a multiple of the vector width,
    accumulate and overwrite."""
    torch.manual_seed(6)
    T, K, L = 77, 1024, 3
    x = torch.randn(T, K).to(dtype)
    A = (torch.randn(L, r, K) * 0.05).to(dtype)
    Bm = (torch.randn(L, N, r) * 0.05).to(dtype)
    if pattern == "random":
        ids = torch.randint(-1, L, (T,), dtype=torch.int32)
    else:   # runs of one adapter: 20 tokens of adapter 1, 20 base-model rows, 30 of adapter 0, 7 of adapter 2
        ids = torch.tensor([1] * 20 + [-1] * 20 + [0] * 30 + [2] * 7, dtype=torch.int32)
    h_ref = ref.bgmv_shrink(x, A, ids, 0.5)
    h = ops.lora_shrink(x.to(DEV), A.to(DEV), ids.to(DEV), 0.5)
    torch.testing.assert_close(h.cpu(), h_ref, atol=2e-3, rtol=2e-3)
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
    for add in (True, False):
        out0 = torch.randn(T, N + offset + 3).to(dtype)
        want = ref.bgmv_expand(h_ref, Bm, ids, out0.clone(), offset=offset, add=add)
        got = ops.lora_expand(h, Bm.to(DEV), ids.to(DEV), out0.to(DEV), offset=offset, add=add)
        torch.testing.assert_close(got.cpu().float(), want.float(), **tol)


def test_mtp_concat_norm_and_sigmoid_gate():
    torch.manual_seed(7)
    T, H = 9, 1024
    e, h = torch.randn(T, H).to(torch.bfloat16), torch.randn(T, H).to(torch.bfloat16)
    we, wh = torch.rand(H).to(torch.bfloat16), torch.rand(H).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 2, 0, 5, 6, 7, 0, 1])
    want = ops.mtp_concat_norm(e, h, we, wh, 1e-6, pos)
    got = ops.mtp_concat_norm(e.to(DEV), h.to(DEV), we.to(DEV), wh.to(DEV), 1e-6, pos.to(DEV))
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)
    wide = torch.randn(T, 3 * H).to(torch.bfloat16)
    o = torch.randn(T, H).to(torch.bfloat16)
    want = ops.sigmoid_gate_mul(o, wide[:, :H])
    got = ops.sigmoid_gate_mul(o.to(DEV), wide.to(DEV)[:, :H])
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)


def _first_logits(llm, prompt):
    from vllm_kunlun_b200 import SamplingParams
    from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
    eng = llm.engine
    eng.add_request(prompt, SamplingParams(max_tokens=1))
    sched = eng.scheduler.schedule()
    md, ids, _ = eng.runner.prepare(sched)
    lora = None if eng.runner.lora is None else eng.runner.lora.punica
    with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate, lora=lora)):
        h, _ = eng.runner.model(ids)
        return eng.runner.model.compute_logits(h[-1:]).float().cpu()


def test_hybrid_engine_on_gpu():
    import dataclasses

    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import qwen3_next_80b_a3b, tiny
    cfg = tiny(qwen3_next_80b_a3b(), num_layers=4, vocab_size=2048, hidden_size=512, num_heads=8, num_kv_heads=2,
               head_dim=64, rotary_dim=16, intermediate_size=512, num_experts=4, num_experts_per_tok=4,  # no routing ties
               moe_intermediate_size=256, gdn_num_k_heads=2, gdn_num_v_heads=4, gdn_head_k_dim=64, gdn_head_v_dim=64,
               max_position=1024)
    kw = dict(block_size=16, max_model_len=512, max_num_seqs=4, num_gpu_blocks=128, max_num_batched_tokens=256)
    gpu = LLM(cfg, device="cuda", enforce_eager=True, **kw)
    cpu = LLM(dataclasses.replace(cfg, dtype="float32"), device="cpu", **kw)
    sd = {k: v.float().cpu() for k, v in gpu.engine.runner.model.state_dict().items()}
    with torch.inference_mode():
        cpu.engine.runner.model.load_state_dict(sd)
    prompt = torch.randint(0, 2048, (150,), generator=torch.Generator().manual_seed(0)).tolist()
    cos = torch.nn.functional.cosine_similarity(_first_logits(gpu, prompt), _first_logits(cpu, prompt)).item()
    assert cos > 0.99, cos
    prompts = [list(range(3, 70)), list(range(100, 117)), list(range(200, 203))]
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    outs = []
    for eager in (True, False):
        llm = LLM(cfg, device="cuda", enforce_eager=eager, seed=5, **kw)
        outs.append([o.token_ids for o in llm.generate(prompts, sp)])
    assert outs[0] == outs[1]


def test_lora_engine_on_gpu():
    import dataclasses

    from test_lora_cpu import _adapter, _cfg
    from vllm_kunlun_b200 import LLM, SamplingParams
    cfg = dataclasses.replace(_cfg(512, 8, 2, 64, 1024, 2048), dtype="bfloat16")
    kw = dict(block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32, enable_lora=True, max_loras=2,
              max_lora_rank=8)
    reqs = [_adapter(cfg, 1), _adapter(cfg, 2, r=8, alpha=4.0, targets=("k_proj", "up_proj", "o_proj")), None]
    gpu = LLM(cfg, device="cuda", enforce_eager=True, **kw)
    cpu = LLM(dataclasses.replace(cfg, dtype="float32"), device="cpu", **kw)
    sd = {k: v.float().cpu() for k, v in gpu.engine.runner.model.state_dict().items()}
    with torch.inference_mode():
        cpu.engine.runner.model.load_state_dict(sd)
    for llm in (gpu, cpu):
        llm.add_lora(reqs[0])
    prompt = list(range(3, 60))
    for llm in (gpu, cpu):
        llm.engine.add_request([1, 2, 3], SamplingParams(max_tokens=1), lora_id=-1)  # a base-model row in the same step
    a, b = [], []
    for llm, dst in ((gpu, a), (cpu, b)):
        eng = llm.engine
        eng.add_request(prompt, SamplingParams(max_tokens=1), lora_id=1)
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
        with torch.inference_mode(), set_forward_context(
                ForwardContext(md, eng.runner.kv_caches, eng.pstate, lora=eng.runner.lora.punica)):
            h, _ = eng.runner.model(ids)
            dst.append(eng.runner.model.compute_logits(h[-1:]).float().cpu())
    cos = torch.nn.functional.cosine_similarity(a[0], b[0]).item()
    assert cos > 0.99, cos
    prompts = [list(range(3, 20)), list(range(30, 41)), list(range(50, 58))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    outs = []
    for eager in (True, False):
        llm = LLM(cfg, device="cuda", enforce_eager=eager, seed=2, **kw)
        outs.append([o.token_ids for o in llm.generate(prompts, sp, lora_request=reqs)])
    assert outs[0] == outs[1]
    base = LLM(cfg, device="cuda", enforce_eager=True, seed=2, **{k: v for k, v in kw.items() if "lora" not in k})
    assert [o.token_ids for o in base.generate(prompts[2:], sp)] == outs[0][2:]


@pytest.mark.parametrize("D", [64, 80, 128])
def test_varlen_bidirectional_attention(D):
    torch.manual_seed(8)
    H = 4
    cu = torch.tensor([0, 100, 100, 357, 400], dtype=torch.int32)
    T = int(cu[-1])
    q, k, v = (torch.randn(T, H, D).to(torch.bfloat16) for _ in range(3))
    want = ops.varlen_attention(q, k, v, cu)
    got = ops.varlen_attention(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV))
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)


def test_qwen_vl_engine_on_gpu():
    import dataclasses

    from test_vision_cpu import IMG, _qwen_vl
    from vllm_kunlun_b200 import LLM, SamplingParams
    cfg = _qwen_vl()
    cfg = dataclasses.replace(cfg, hidden_size=512, num_heads=8, num_kv_heads=2, head_dim=64, v_head_dim=64, rotary_dim=64,
                              intermediate_size=1024, vocab_size=2048, dtype="bfloat16", mrope_section=(8, 12, 12))
    cfg.vision = dict(cfg.vision, hidden=128, heads=2, intermediate=256, patch=4, image_token_id=2047)
    grid = [(1, 16, 8)]
    px = torch.randn(128, 3 * 1 * 4 * 4, generator=torch.Generator().manual_seed(0))
    prompt = [5, 6, 7] + [2047] * 32 + [9, 10, 11, 12]
    kw = dict(block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64)
    gpu = LLM(cfg, device="cuda", enforce_eager=True, **kw)
    cpu = LLM(dataclasses.replace(cfg, dtype="float32"), device="cpu", **kw)
    sd = {k: v.float().cpu() for k, v in gpu.engine.runner.model.state_dict().items()}
    with torch.inference_mode():
        cpu.engine.runner.model.load_state_dict(sd)
    mm = {"pixel_values": px, "image_grid_thw": grid}
    ea = gpu.engine.runner.model.embed_multimodal(px, grid).float().cpu()
    eb = cpu.engine.runner.model.embed_multimodal(px, grid).float()
    assert torch.nn.functional.cosine_similarity(ea.flatten(), eb.flatten(), dim=0) > 0.99

    def logits(llm):
        from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
        eng = llm.engine
        eng.add_request(prompt, SamplingParams(max_tokens=1), multi_modal_data=mm)
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        ctx = ForwardContext(md, eng.runner.kv_caches, eng.pstate, extras=eng.runner._step_extras)
        with torch.inference_mode(), set_forward_context(ctx):
            h, _ = eng.runner.model(ids)
            return eng.runner.model.compute_logits(h[-1:]).float().cpu()

    cos = torch.nn.functional.cosine_similarity(logits(gpu), logits(cpu)).item()
    assert cos > 0.99, cos
    out = LLM(cfg, device="cuda", **kw).generate([prompt], SamplingParams(max_tokens=5, ignore_eos=True), multi_modal_data=mm)
    assert len(out[0].token_ids) == 5

