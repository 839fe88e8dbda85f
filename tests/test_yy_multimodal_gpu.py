"""Whole multimodal models on the GPU against their fp32 CPU twins: Gemma-4 (sparse block beside the MLP, vision
tower) and the Qwen3-Omni audio encoder.  Collected after the kernel and engine suites because each test builds
complete models on both devices."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _prefill_logits(llm, prompt, mm=None):
    from vllm_kunlun_b200 import SamplingParams
    from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
    eng = llm.engine
    eng.add_request(prompt, SamplingParams(max_tokens=1), multi_modal_data=mm)
    md, ids, _ = eng.runner.prepare(eng.scheduler.schedule())
    ctx = ForwardContext(md, eng.runner.kv_caches, eng.pstate, extras=eng.runner._step_extras)
    with torch.inference_mode(), set_forward_context(ctx):
        h, _ = eng.runner.model(ids)
        return eng.runner.model.compute_logits(h[-1:]).float().cpu()


def test_gemma4_sparse_block_and_vision_tower_on_gpu():
    """Gemma-4 with the sparse block beside the MLP and an image in the prompt: bf16 on the GPU against the fp32 CPU
    model holding the same weights (router kernel with fp32 scores, tanh-GELU experts, 2-D rotary tower)."""
    import dataclasses

    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import ModelConfig
    IMG = 500
    d = dict(architectures=["Gemma4ForConditionalGeneration"], image_token_id=IMG, torch_dtype="bfloat16",
             text_config=dict(vocab_size=512, hidden_size=256, num_hidden_layers=4,
                              layer_types=["sliding_attention", "full_attention"] * 2, num_attention_heads=4,
                              num_key_value_heads=2, head_dim=64, global_head_dim=64, intermediate_size=512,
                              max_position_embeddings=256, sliding_window=16, hidden_size_per_layer_input=0,
                              num_kv_shared_layers=0, enable_moe_block=True, num_experts=8, top_k_experts=2,
                              moe_intermediate_size=128, rms_norm_eps=1e-6),
             vision_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                                num_key_value_heads=2, head_dim=64, patch_size=4, position_embedding_size=32,
                                pooling_kernel_size=2))
    cfg = ModelConfig.from_hf_config(d)
    kw = dict(block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64)
    gpu = LLM(cfg, device="cuda", enforce_eager=True, **kw)
    cpu = LLM(dataclasses.replace(cfg, dtype="float32"), device="cpu", **kw)
    sd = {k: v.float().cpu() for k, v in gpu.engine.runner.model.state_dict().items()}
    with torch.inference_mode():
        cpu.engine.runner.model.load_state_dict(sd)
    grid = [(1, 8, 4)]
    px = torch.rand(32, 3 * 16, generator=torch.Generator().manual_seed(0))
    ea = gpu.engine.runner.model.embed_multimodal(px, grid).float().cpu()
    eb = cpu.engine.runner.model.embed_multimodal(px, grid).float()
    assert ea.shape == (8, 256) and torch.nn.functional.cosine_similarity(ea.flatten(), eb.flatten(), dim=0) > 0.99
    prompt = [5, 6, 7] + [IMG] * 8 + [9, 10, 11, 12]
    mm = {"pixel_values": px, "image_grid_thw": grid}
    # the decoder is compared on identical soft tokens: with unit norm weights and softmax scale 1 the random-weight
    # attention is nearly one-hot, which turns the tower's bf16 rounding into different attention targets
    gpu.engine.runner.model.embed_multimodal = lambda pixels, grids: eb.to(DEV, torch.bfloat16)
    cos = torch.nn.functional.cosine_similarity(_prefill_logits(gpu, prompt, mm), _prefill_logits(cpu, prompt, mm)).item()
    assert cos > 0.99, cos
    out = LLM(cfg, device="cuda", enforce_eager=True, **kw).generate(
        [prompt], SamplingParams(max_tokens=5, ignore_eos=True), multi_modal_data=mm)
    assert len(out[0].token_ids) == 5


def test_qwen3_omni_audio_tower_on_gpu():
    """The audio encoder (convolution stem, windowed attention, projection) in bf16 on the GPU against fp32 on the
    CPU, two clips, one of them longer than an attention window."""
    from vllm_kunlun_b200.models.omni import AudioEncoder
    ac = dict(hidden=128, heads=2, intermediate=256, depth=2, n_mels=32, n_window=50, n_window_infer=200,
              downsample_hidden=16)
    torch.manual_seed(0)
    cpu = AudioEncoder(ac, 256, torch.float32, "cpu")
    for n, p in cpu.named_parameters():
        p.data.copy_(torch.ones_like(p) if (p.dim() == 1 and "norm" in n or n.endswith("ln_post.weight"))
                     else torch.randn_like(p) * (0.3 if "conv" in n else 0.05))
    gpu = AudioEncoder(ac, 256, torch.bfloat16, DEV)
    with torch.inference_mode():
        gpu.load_state_dict({k: v.to(torch.bfloat16) for k, v in cpu.state_dict().items()})
        lens = [430, 70]
        feats = torch.randn(sum(lens), 32)
        want = cpu(feats, lens)
        got = gpu(feats.to(DEV), lens).float().cpu()
    assert got.shape == want.shape == (sum(cpu.output_lengths(lens)), 256)
    assert torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0) > 0.99


def test_chunked_gated_delta_rule_on_gpu(monkeypatch):
    """``B200_GDN_CHUNKED=1``: a 300-token request takes the chunked form (batched products on the GPU), a decode
    row and a short request keep the recurrent kernel; outputs and states equal the fp32 token-by-token rule."""
    from vllm_kunlun_b200 import ops
    from vllm_kunlun_b200.ops.reference import misc as ref
    torch.manual_seed(0)
    lens = [300, 1, 40]
    L, Hk, Hv, Dk, Dv = sum(lens), 2, 4, 128, 128
    q, k = torch.randn(L, Hk, Dk).bfloat16(), torch.randn(L, Hk, Dk).bfloat16()
    v = torch.randn(L, Hv, Dv).bfloat16()
    g, beta = -torch.rand(L, Hv) * 0.3, torch.rand(L, Hv)
    cu = torch.tensor([0, 300, 301, 341], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    has = torch.tensor([True, True, False])
    base = torch.randn(5, Hv, Dv, Dk) * 0.1
    want, want_st = torch.empty(L, Hv, Dv), base.clone()
    for r in range(3):
        s, e, slot = int(cu[r]), int(cu[r + 1]), int(slots[r])
        S0 = base[slot] if bool(has[r]) else torch.zeros_like(base[slot])
        o, S = ref.recurrent_gated_delta_rule(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e], S0)
        want[s:e], want_st[slot] = o.float(), S
    monkeypatch.setenv("B200_GDN_CHUNKED", "1")
    st = base.to(DEV)
    got = ops.gated_delta_rule(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), st, cu.to(DEV), slots.to(DEV),
                               has.to(DEV), None, True, cu.clone())
    torch.testing.assert_close(got.float().cpu(), want, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(st.cpu(), want_st, atol=2e-2, rtol=2e-2)
