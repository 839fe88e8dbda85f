"""Gemma-family (sandwich norms, KV sharing) and MiMo-V2-Flash (narrow value heads) on the CPU oracle path."""
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import ModelConfig, llama_3_1_8b, qwen3_30b_a3b, tiny
from vllm_kunlun_b200.models.gemma4 import kv_source_layer

KW = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=48)


def _gemma():
    cfg = tiny(llama_3_1_8b(), num_layers=6, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    cfg.architecture = "Gemma4ForCausalLM"
    cfg.gemma_norm, cfg.qk_norm, cfg.hidden_act, cfg.tie_word_embeddings = True, True, "gelu_tanh", True
    cfg.sliding_window, cfg.sliding_window_pattern = 8, 3
    cfg.num_kv_shared_layers, cfg.final_logit_softcapping, cfg.attn_scale = 2, 30.0, 1.0
    return cfg


def test_gemma_kv_sharing_layout_and_generation():
    cfg = _gemma()
    # layers 0,1 sliding, 2 full, 3,4 sliding, 5 full; the last two share: 4 -> 3 (sliding), 5 -> 2 (full)
    assert [kv_source_layer(cfg, i) for i in range(6)] == [0, 1, 2, 3, 3, 2]
    llm = LLM(cfg, max_num_batched_tokens=64, **KW)
    assert sorted(llm.engine.runner.kv_caches) == [0, 1, 2, 3]
    prompts = [list(range(3, 40)), list(range(50, 57))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = [o.token_ids for o in llm.generate(prompts, sp)]
    b = [o.token_ids for o in LLM(cfg, max_num_batched_tokens=16, **KW).generate(prompts, sp)]
    assert a == b
    lg = llm.engine.runner.model.compute_logits(torch.randn(2, 64) * 100)
    assert lg.abs().max() <= 30.0


def test_mimo_narrow_value_heads_are_padded_in_the_weights():
    cfg = tiny(qwen3_30b_a3b(fp8=False), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=2,
               head_dim=32, v_head_dim=16, intermediate_size=128, num_experts=4, num_experts_per_tok=2,
               moe_intermediate_size=64, max_position=256, dtype="float32")
    cfg.architecture = "MiMoV2FlashForCausalLM"
    cfg.attention_sinks, cfg.sliding_window = True, 16
    llm = LLM(cfg, **KW)
    m = llm.engine.runner.model
    g = torch.Generator().manual_seed(0)
    H, D, Dv, hid = 2, 32, 16, 64
    ck = {"model.layers.0.self_attn.q_proj.weight": torch.randn(H * D, hid, generator=g),
          "model.layers.0.self_attn.k_proj.weight": torch.randn(H * D, hid, generator=g),
          "model.layers.0.self_attn.v_proj.weight": torch.randn(H * Dv, hid, generator=g),
          "model.layers.0.self_attn.o_proj.weight": torch.randn(hid, H * Dv, generator=g),
          "model.layers.0.self_attn.attention_sink_bias": torch.randn(H, generator=g)}
    with torch.inference_mode():
        m.load_weights(ck.items())
    qkv = m.layers["0"].self_attn.qkv_proj.weight.data
    v = qkv[2 * H * D:].reshape(H, D, hid)
    assert torch.equal(v[:, :Dv].reshape(H * Dv, hid), ck["model.layers.0.self_attn.v_proj.weight"])
    assert v[:, Dv:].abs().sum() == 0
    o = m.layers["0"].self_attn.o_proj.weight.data.reshape(hid, H, D)
    assert torch.equal(o[:, :, :Dv].reshape(hid, H * Dv), ck["model.layers.0.self_attn.o_proj.weight"])
    assert o[:, :, Dv:].abs().sum() == 0
    assert torch.equal(m.layers["0"].self_attn.sinks.data, ck["model.layers.0.self_attn.attention_sink_bias"])
    # padded-weight attention equals attention with narrow V followed by the narrow o_proj
    x = torch.randn(5, hid, generator=g)
    attn = m.layers["0"].self_attn
    vv = (x @ qkv[2 * H * D:].T).reshape(5, H, D)
    narrow = (vv[:, :, :Dv].reshape(5, H * Dv) @ ck["model.layers.0.self_attn.o_proj.weight"].T)
    padded = vv.reshape(5, H * D) @ attn.o_proj.weight.data.T
    torch.testing.assert_close(narrow, padded)
    out = llm.generate([list(range(3, 30))], SamplingParams(max_tokens=4, ignore_eos=True))
    assert len(out[0].token_ids) == 4


def test_mimo_fp8_attention_weights_are_dequantised_on_load():
    from vllm_kunlun_b200.models.mimo_v2_flash import _dequant_block
    from vllm_kunlun_b200.models.moe import _quant_block_device
    w = torch.randn(256, 256)
    q, s = _quant_block_device(w)
    torch.testing.assert_close(_dequant_block(q, s), w, atol=0.15, rtol=0.1)


def test_gpt_oss_checkpoint_layout():
    from vllm_kunlun_b200.config import gpt_oss_20b
    cfg = tiny(gpt_oss_20b(), num_layers=2, vocab_size=128, hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16,
               intermediate_size=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, max_position=256,
               dtype="float32")
    llm = LLM(cfg, **KW)
    m = llm.engine.runner.model
    g = torch.Generator().manual_seed(0)
    E, H, I = 4, 64, 32
    gu = torch.randn(E, H, 2 * I, generator=g)
    gub = torch.randn(E, 2 * I, generator=g)
    dn = torch.randn(E, I, H, generator=g)
    dnb = torch.randn(E, H, generator=g)
    sinks = torch.randn(4, generator=g)
    router = torch.randn(E, H, generator=g)
    ck = {"model.layers.1.mlp.experts.gate_up_proj": gu, "model.layers.1.mlp.experts.gate_up_proj_bias": gub,
          "model.layers.1.mlp.experts.down_proj": dn, "model.layers.1.mlp.experts.down_proj_bias": dnb,
          "model.layers.1.self_attn.sinks": sinks, "model.layers.1.mlp.router.weight": router,
          "model.layers.1.mlp.router.bias": torch.zeros(E)}
    with torch.inference_mode():
        loaded = m.load_weights(ck.items())
    assert {n.replace('.mlp.gate.', '.mlp.router.') for n in loaded} == set(ck)
    ex = m.layers["1"].mlp.experts
    x = torch.randn(3, H, generator=g)
    e = 2
    h = x @ gu[e] + gub[e]                                   # checkpoint semantics: interleaved gate / up
    gate, up = h[:, 0::2], h[:, 1::2]
    mine = x @ ex.w13.data[e].T + ex.b13.data[e]
    # the expert weights keep the interleaved order the family's activation reads
    torch.testing.assert_close(mine[:, 0::2], gate, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(mine[:, 1::2], up, atol=1e-5, rtol=1e-5)
    a = torch.randn(3, I, generator=g)
    torch.testing.assert_close(a @ ex.w2.data[e].T + ex.b2.data[e], a @ dn[e] + dnb[e], atol=1e-5, rtol=1e-5)
    assert torch.equal(m.layers["1"].self_attn.sinks.data, sinks)
    assert torch.equal(m.layers["1"].mlp.gate.weight.data, router)
    assert len(llm.generate([list(range(3, 40))], SamplingParams(max_tokens=4, ignore_eos=True))[0].token_ids) == 4


def test_gemma_per_layer_inputs_and_multimodal():
    """Per-layer inputs change the output and follow the reference arithmetic; the multimodal wrapper replaces
    placeholder rows after the embedding scale and survives chunked prefill."""
    cfg = _gemma()
    cfg.num_kv_shared_layers = 0
    cfg.per_layer_input_size, cfg.per_layer_vocab_size = 8, 100
    llm = LLM(cfg, max_num_batched_tokens=64, **KW)
    m = llm.engine.runner.model
    L, P, H = cfg.num_layers, 8, cfg.hidden_size
    assert m.embed_tokens_per_layer.weight.shape == (128, L * P)  # vocab padded to 64-row shards
    assert all(float(layer.layer_scalar) == 1.0 for layer in m.layers.values())
    ids = torch.tensor([3, 99, 120, 7])           # 120 is outside the per-layer vocabulary: looks up row 0
    emb = torch.randn(4, H, generator=torch.Generator().manual_seed(0))
    ple = m.per_layer_inputs(ids, emb)
    assert ple.shape == (4, L, P)
    tok = m.embed_tokens_per_layer.weight[torch.tensor([3, 99, 0, 7])].view(4, L, P) * P ** 0.5
    proj = (emb @ m.per_layer_model_projection.weight.T * H ** -0.5).view(4, L, P)
    w = m.per_layer_projection_norm.weight
    proj = proj * torch.rsqrt(proj.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * (1 + w)
    torch.testing.assert_close(ple, (proj + tok) * 2 ** -0.5, atol=1e-5, rtol=1e-4)
    prompts = [list(range(3, 30))]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    a = llm.generate(prompts, sp)[0].token_ids
    assert a == LLM(cfg, max_num_batched_tokens=8, **KW).generate(prompts, sp)[0].token_ids
    plain = _gemma()
    plain.num_kv_shared_layers = 0
    assert LLM(plain, max_num_batched_tokens=64, **KW).engine.runner.model.ple == 0
    # multimodal wrapper
    IMG = 127
    cfg.architecture = "Gemma4ForConditionalGeneration"
    cfg.vision = dict(depth=2, hidden=32, heads=2, patch=2, intermediate=64, in_channels=3, pool=2,
                      position_embedding_size=16, image_token_id=IMG)
    vl = LLM(cfg, max_num_batched_tokens=64, **KW)
    tower = vl.engine.runner.model.visual
    assert tower.tokens_per_image((1, 4, 4)) == 4
    px = torch.rand(1, 16, 12, generator=torch.Generator().manual_seed(1))      # a 4 x 4 grid of 2 x 2-pixel patches
    assert vl.engine.runner.model.embed_multimodal(px).shape == (4, H)
    prompt = [5, 6] + [IMG] * 4 + [9, 10, 11]
    o1 = vl.generate([prompt], sp, multi_modal_data={"pixel_values": px})[0].token_ids
    o2 = LLM(cfg, max_num_batched_tokens=4, **KW).generate([prompt], sp, multi_modal_data={"pixel_values": px})[0].token_ids
    assert o1 == o2 and len(o1) == 5
