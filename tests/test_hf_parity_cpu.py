"""Model families against the Hugging Face reference implementations (CPU, fp32, tiny random-weight instances).

For every family: build the ``transformers`` model from a small config, randomise its weights, take the logits of a
prompt; build this package's model from the SAME config dict (``ModelConfig.from_hf_config``), load the SAME state
dict through the model's checkpoint loader, run the prompt through the engine's prefill path and compare the logits.
This checks the config parsing, the checkpoint name mapping / stacking / expert layouts and the model mathematics
(attention variants, rotary variants, routing rules, activations) in one go.
"""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from vllm_kunlun_b200 import LLM, SamplingParams  # noqa: E402
from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context  # noqa: E402
from vllm_kunlun_b200.config import ModelConfig  # noqa: E402

COMMON = dict(vocab_size=160, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=256, max_position_embeddings=256, rms_norm_eps=1e-5)
DS = dict(vocab_size=160, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
          intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8, num_experts_per_tok=2,
          first_k_dense_replace=1, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
          max_position_embeddings=256, rms_norm_eps=1e-5)
GPT_OSS = dict(vocab_size=160, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               head_dim=32, intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=256)
Q35 = dict(vocab_size=160, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
           intermediate_size=256, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
           linear_value_head_dim=32, linear_conv_kernel_dim=4, full_attention_interval=4, max_position_embeddings=256)
GEMMA4 = dict(vocab_size=160, hidden_size=128, num_hidden_layers=6, layer_types=["sliding_attention", "full_attention"] * 3,
              num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, max_position_embeddings=256,
              sliding_window=8)
YARN = {"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "original_max_position_embeddings": 64,
        "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0}

# (id, transformers config class, transformers model class, architecture string, config arguments, tolerance)
CASES = [
    ("llama", "LlamaConfig", "LlamaForCausalLM", "LlamaForCausalLM", dict(COMMON, rope_theta=500000.0), 1e-4),
    ("llama3_rope_scaling", "LlamaConfig", "LlamaForCausalLM", "LlamaForCausalLM",
     dict(COMMON, rope_theta=500000.0, rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64}), 1e-4),
    ("mistral_sliding_window", "MistralConfig", "MistralForCausalLM", "MistralForCausalLM", dict(COMMON, sliding_window=8), 1e-4),
    ("qwen2_bias", "Qwen2Config", "Qwen2ForCausalLM", "Qwen2ForCausalLM", dict(COMMON), 1e-4),
    ("qwen3_qk_norm", "Qwen3Config", "Qwen3ForCausalLM", "Qwen3ForCausalLM", dict(COMMON, head_dim=48), 1e-4),
    ("seed_oss", "SeedOssConfig", "SeedOssForCausalLM", "SeedOssForCausalLM", dict(COMMON, head_dim=32), 1e-4),
    ("mixtral", "MixtralConfig", "MixtralForCausalLM", "MixtralForCausalLM",
     dict(COMMON, num_local_experts=4, num_experts_per_tok=2), 1e-4),
    ("qwen3_moe", "Qwen3MoeConfig", "Qwen3MoeForCausalLM", "Qwen3MoeForCausalLM",
     dict(COMMON, head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
          decoder_sparse_step=1, mlp_only_layers=[]), 1e-4),
    ("qwen2_moe_shared_expert", "Qwen2MoeConfig", "Qwen2MoeForCausalLM", "Qwen2MoeForCausalLM",
     dict(COMMON, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=96,
          norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[]), 1e-4),
    ("glm4_moe", "Glm4MoeConfig", "Glm4MoeForCausalLM", "Glm4MoeForCausalLM",
     dict(vocab_size=160, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
          intermediate_size=256, attention_bias=True, partial_rotary_factor=0.5, use_qk_norm=True, n_routed_experts=8,
          n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=64, first_k_dense_replace=1, n_group=1,
          topk_group=1, routed_scaling_factor=1.5, norm_topk_prob=True, max_position_embeddings=256, rms_norm_eps=1e-5), 1e-4),
    ("deepseek_v3_mla_sigmoid_groups", "DeepseekV3Config", "DeepseekV3ForCausalLM", "DeepseekV3ForCausalLM",
     dict(DS, q_lora_rank=64, n_shared_experts=1, n_group=2, topk_group=1, routed_scaling_factor=2.5, norm_topk_prob=True), 5e-4),
    ("deepseek_v3_yarn", "DeepseekV3Config", "DeepseekV3ForCausalLM", "DeepseekV3ForCausalLM",
     dict(DS, q_lora_rank=64, n_shared_experts=1, n_group=2, topk_group=1, routed_scaling_factor=2.5, norm_topk_prob=True,
          rope_parameters=YARN), 5e-4),
    ("deepseek_v3_plain_q_proj", "DeepseekV3Config", "DeepseekV3ForCausalLM", "DeepseekV3ForCausalLM",
     dict(DS, q_lora_rank=None, n_shared_experts=1, n_group=2, topk_group=1, routed_scaling_factor=2.5, norm_topk_prob=True), 5e-4),
    ("deepseek_v2_softmax_routing", "DeepseekV2Config", "DeepseekV2ForCausalLM", "DeepseekV2ForCausalLM",
     dict(DS, q_lora_rank=None, n_shared_experts=2, n_group=1, topk_group=1, routed_scaling_factor=1.0, norm_topk_prob=False,
          topk_method="greedy"), 5e-4),
    ("gpt_oss_sinks_swa_yarn", "GptOssConfig", "GptOssForCausalLM", "GptOssForCausalLM",
     dict(GPT_OSS, sliding_window=8, layer_types=["sliding_attention", "full_attention"]), 1e-4),
    ("gpt_oss_plain_rope", "GptOssConfig", "GptOssForCausalLM", "GptOssForCausalLM",
     dict(GPT_OSS, sliding_window=64, rope_parameters={"rope_type": "default", "rope_theta": 150000.0},
          layer_types=["full_attention", "full_attention"]), 1e-4),
    ("qwen3_next_gated_delta_net", "Qwen3NextConfig", "Qwen3NextForCausalLM", "Qwen3NextForCausalLM",
     dict(vocab_size=160, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
          intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=64, num_experts=4,
          num_experts_per_tok=2, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
          linear_value_head_dim=32, linear_conv_kernel_dim=4, full_attention_interval=4, partial_rotary_factor=0.25,
          max_position_embeddings=256, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[]), 5e-4),
    ("qwen3_5_dense_hybrid", "Qwen3_5TextConfig", "Qwen3_5ForCausalLM", "Qwen3_5ForCausalLM", dict(Q35), 5e-4),
    ("qwen3_5_moe_hybrid", "Qwen3_5MoeTextConfig", "Qwen3_5MoeForCausalLM", "Qwen3_5MoeForCausalLM",
     dict(Q35, moe_intermediate_size=64, shared_expert_intermediate_size=64, num_experts=4, num_experts_per_tok=2), 5e-4),
    # Gemma-4: sandwich norms with plain weights, softmax scale 1, V norm, layer scalars, per-type rotary parameters
    ("gemma4_basic", "Gemma4TextConfig", "Gemma4ForCausalLM", "Gemma4ForCausalLM",
     dict(GEMMA4, global_head_dim=32, hidden_size_per_layer_input=0, num_kv_shared_layers=0), 1e-4),
    # ... plus proportional rotary embedding and a larger head on the full-attention layers whose values are their keys,
    # per-layer inputs, cross-layer KV sharing with double-wide MLPs
    ("gemma4_full_featured", "Gemma4TextConfig", "Gemma4ForCausalLM", "Gemma4ForCausalLM",
     dict(GEMMA4, global_head_dim=64, attention_k_eq_v=True, num_global_key_value_heads=1, hidden_size_per_layer_input=64,
          vocab_size_per_layer_input=160, num_kv_shared_layers=2, use_double_wide_mlp=True,
          rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                           "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                                              "rope_theta": 1000000.0}}), 1e-4),
    # ... and the sparse block beside every dense MLP (own router: scale-free norm, per-channel and per-expert scales)
    ("gemma4_moe_block", "Gemma4TextConfig", "Gemma4ForCausalLM", "Gemma4ForCausalLM",
     dict(GEMMA4, global_head_dim=32, hidden_size_per_layer_input=0, num_kv_shared_layers=0, enable_moe_block=True,
          num_experts=4, top_k_experts=2, moe_intermediate_size=64), 1e-4),
    # GLM-MoE-DSA (DeepSeek-V3.2 style sparse attention): with a top-k above the prompt length every key is selected,
    # so the whole path (indexer, index conversion, sparse MLA) must reproduce dense attention
    ("glm_moe_dsa_indexer", "GlmMoeDsaConfig", "GlmMoeDsaForCausalLM", "GlmMoeDsaForCausalLM",
     dict(DS, q_lora_rank=64, n_shared_experts=1, n_group=1, topk_group=1, index_topk=64, index_n_heads=4,
          index_head_dim=128, mlp_layer_types=["dense", "sparse", "sparse"]), 5e-4),
]


def _randomise(model):
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name and p.dim() == 1:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.05)
            else:
                p.copy_(torch.randn_like(p) * 0.1)      # biases, sinks, router correction biases


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_logits_match_the_transformers_implementation(case):
    _, cfg_name, cls_name, arch, kwargs, tol = case
    if not (hasattr(transformers, cfg_name) and hasattr(transformers, cls_name)):
        pytest.skip(f"transformers {transformers.__version__} has no {cls_name}")
    torch.manual_seed(0)
    hf_cfg = getattr(transformers, cfg_name)(**kwargs)
    hf_cfg._attn_implementation = "eager"      # the plain-PyTorch attention of the reference implementation
    hf = getattr(transformers, cls_name)(hf_cfg).eval().float()
    _randomise(hf)
    ids = torch.randint(1, hf_cfg.vocab_size - 1, (1, 19))
    with torch.no_grad():
        want = hf(ids).logits[0].float()
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = [arch], "float32"
    cfg = ModelConfig.from_hf_config(d)
    llm = LLM(cfg, device="cpu", block_size=64 if cfg.index_topk else 16, max_model_len=128, max_num_seqs=4,
              num_gpu_blocks=32)
    model = llm.engine.runner.model
    with torch.inference_mode():
        loaded = model.load_weights(list(hf.state_dict().items()))
    assert len(loaded) >= len(hf.state_dict()) - 12, "most checkpoint tensors must find their parameter"
    eng = llm.engine
    eng.add_request(ids[0].tolist(), SamplingParams(max_tokens=1))
    md, tok, _ = eng.runner.prepare(eng.scheduler.schedule())
    with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
        h, _ = model(tok)
        got = model.compute_logits(h).float()
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"{case[0]}: max |logit difference| {err:.3g}"
    # and the engine's own path (scheduler, KV cache, sampler): greedy continuation = the reference's argmax chain
    out = llm.generate([ids[0].tolist()], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))[0].token_ids
    seq = ids.clone()
    with torch.no_grad():
        for _ in range(3):
            nxt = hf(seq).logits[0, -1].argmax().view(1, 1)
            seq = torch.cat([seq, nxt], 1)
    assert out == seq[0, -3:].tolist()


_TOK = dict(image_token_id=150, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153)
VL_CASES = [
    # Qwen2-VL: LayerNorm blocks, quick-GELU MLP, full attention per frame, M-RoPE decoder
    ("qwen2_vl", "Qwen2VLConfig", "Qwen2VLForConditionalGeneration", "Qwen2VLForConditionalGeneration",
     dict(rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]}),
     dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=4, spatial_merge_size=2,
          temporal_patch_size=2, in_channels=3)),
    # Qwen2.5-VL: RMSNorm blocks, gated MLP (gate / up / down tensors), windowed attention except in listed blocks.
    # tokens_per_second=1: transformers 5 multiplies an image's temporal position by tokens_per_second (the model's
    # own rule, followed here, scales only the frame index of a video, so an image keeps its start position).
    ("qwen2_5_vl_windows", "Qwen2_5_VLConfig", "Qwen2_5_VLForConditionalGeneration", "Qwen2_5_VLForConditionalGeneration",
     dict(rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]}),
     dict(depth=3, hidden_size=64, out_hidden_size=128, num_heads=4, intermediate_size=128, patch_size=4,
          spatial_merge_size=2, temporal_patch_size=2, in_channels=3, window_size=16, fullatt_block_indexes=[1],
          tokens_per_second=1)),
    # Qwen3-VL: patch bias, interpolated position table, tanh-GELU MLP, deep-stack features, interleaved M-RoPE
    ("qwen3_vl_deepstack", "Qwen3VLConfig", "Qwen3VLForConditionalGeneration", "Qwen3VLForConditionalGeneration",
     dict(head_dim=32, rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True}),
     dict(depth=3, hidden_size=64, out_hidden_size=128, num_heads=4, intermediate_size=128, patch_size=4,
          spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=64,
          deepstack_visual_indexes=[0, 1])),
    # Qwen3-VL-MoE: the same tower over a sparse decoder with stacked expert tensors
    ("qwen3_vl_moe", "Qwen3VLMoeConfig", "Qwen3VLMoeForConditionalGeneration", "Qwen3VLMoeForConditionalGeneration",
     dict(head_dim=32, moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
          decoder_sparse_step=1, mlp_only_layers=[],
          rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True}),
     dict(depth=3, hidden_size=64, out_hidden_size=128, num_heads=4, intermediate_size=128, patch_size=4,
          spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=64,
          deepstack_visual_indexes=[0, 1])),
]


@pytest.mark.parametrize("case", VL_CASES, ids=[c[0] for c in VL_CASES])
def test_vision_language_models_match_the_transformers_implementation(case):
    """Two images of different grids in one prompt: the vision tower's embeddings (and deep-stack features) equal the
    reference's; the logits after the prompt (placeholder rows replaced during prefill, M-RoPE positions, deep-stack
    injection) equal the reference's, and so do eight greedily decoded tokens."""
    _, cfg_name, cls_name, arch, text_kw, vis_kw = case
    if not (hasattr(transformers, cfg_name) and hasattr(transformers, cls_name)):
        pytest.skip(f"transformers {transformers.__version__} has no {cls_name}")
    torch.manual_seed(0)
    tc = dict(vocab_size=200, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=256, max_position_embeddings=512, rms_norm_eps=1e-5, **text_kw)
    hf_cfg = getattr(transformers, cfg_name)(text_config=tc, vision_config=vis_kw, **_TOK)
    hf = getattr(transformers, cls_name)(hf_cfg).eval().float()
    _randomise(hf)
    vc = hf_cfg.vision_config
    grids = [(1, 8, 12), (1, 4, 6)]
    patch_dim = 3 * vc.temporal_patch_size * vc.patch_size ** 2
    px = torch.randn(sum(t * h * w for t, h, w in grids), patch_dim)
    m2 = vc.spatial_merge_size ** 2
    img = hf_cfg.image_token_id
    ids = [5, 6, 7] + [img] * (8 * 12 // m2) + [8, 9] + [img] * (4 * 6 // m2) + [10, 11, 12]
    gthw = torch.tensor(grids)

    def hf_logits(seq):
        with torch.no_grad():
            return hf(input_ids=seq, pixel_values=px, image_grid_thw=gthw, mm_token_type_ids=(seq == img).long()).logits[0]

    seq = torch.tensor([ids])
    want = []
    want_logits = None
    for _ in range(8):
        lg = hf_logits(seq)[-1].float()
        want_logits = lg if want_logits is None else want_logits
        want.append(lg.argmax().item())
        seq = torch.cat([seq, torch.tensor([[want[-1]]])], 1)
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = [arch], "float32"
    cfg = ModelConfig.from_hf_config(d)
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=32)
    model = llm.engine.runner.model
    with torch.inference_mode():
        loaded = model.load_weights(list(hf.state_dict().items()))
    assert len(loaded) == len(hf.state_dict())
    with torch.no_grad():
        ref = hf.model.visual(px, grid_thw=gthw)
    ref_main = ref.pooler_output if hasattr(ref, "pooler_output") else (ref[0] if isinstance(ref, tuple) else ref)
    deep = getattr(ref, "deepstack_features", None) if not isinstance(ref, tuple) else (ref[1] if len(ref) > 1 else None)
    with torch.inference_mode():
        mine = model.embed_multimodal(px, [list(g) for g in grids]).float()
    H = ref_main.shape[-1]
    assert (mine[:, :H] - ref_main.float()).abs().max().item() < 1e-4
    for k, f in enumerate(deep or []):
        assert (mine[:, (k + 1) * H:(k + 2) * H] - f.float()).abs().max().item() < 1e-4
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    out = llm.generate([ids], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True),
                       multi_modal_data={"pixel_values": px, "image_grid_thw": [list(g) for g in grids]})[0].token_ids
    assert (seen[0][-1] - want_logits).abs().max().item() < 1e-4
    assert out == want


def test_qwen3_vl_image_and_video_prompt_matches_the_transformers_implementation():
    """One image and one two-frame video in a prompt (Qwen3-VL: one video placeholder run per temporal patch, with
    text in between): the logits after the prompt equal the reference's."""
    _, cfg_name, cls_name, arch, text_kw, vis_kw = VL_CASES[2]
    if not (hasattr(transformers, cfg_name) and hasattr(transformers, cls_name)):
        pytest.skip(f"transformers {transformers.__version__} has no {cls_name}")
    torch.manual_seed(0)
    tc = dict(vocab_size=200, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=256, max_position_embeddings=512, rms_norm_eps=1e-5, **text_kw)
    hf_cfg = getattr(transformers, cfg_name)(text_config=tc, vision_config=vis_kw, **_TOK)
    hf = getattr(transformers, cls_name)(hf_cfg).eval().float()
    _randomise(hf)
    img, vid = hf_cfg.image_token_id, hf_cfg.video_token_id
    patch_dim = 3 * hf_cfg.vision_config.temporal_patch_size * hf_cfg.vision_config.patch_size ** 2
    px, pv = torch.randn(1 * 4 * 6, patch_dim), torch.randn(2 * 4 * 4, patch_dim)
    ids = [5, 6] + [img] * 6 + [7, 30, 31] + [vid] * 4 + [32, 33] + [vid] * 4 + [8, 9, 10]
    seq = torch.tensor([ids])
    with torch.no_grad():
        want = hf(input_ids=seq, pixel_values=px, image_grid_thw=torch.tensor([[1, 4, 6]]), pixel_values_videos=pv,
                  video_grid_thw=torch.tensor([[2, 4, 4]]),
                  mm_token_type_ids=(seq == img).long() + 2 * (seq == vid).long()).logits[0, -1].float()
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = [arch], "float32"
    llm = LLM(ModelConfig.from_hf_config(d), device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=32)
    model = llm.engine.runner.model
    with torch.inference_mode():
        model.load_weights(list(hf.state_dict().items()))
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
                 multi_modal_data={"pixel_values": px, "image_grid_thw": [[1, 4, 6]], "pixel_values_videos": pv,
                                   "video_grid_thw": [[2, 4, 4]]})
    assert (seen[0][-1] - want).abs().max().item() < 1e-4


def test_qwen3_omni_thinker_matches_the_transformers_implementation():
    """Audio clip + image in one prompt through the Qwen3-Omni thinker: the audio tower's rows (three-convolution
    stem over 100-frame chunks, tail chunk shorter), and the logits after the prompt (audio rows, image rows with
    deep-stack features, interleaved M-RoPE, sparse decoder) equal the reference's.  The clip fits one attention
    window: the library's non-flash attention paths ignore the window boundaries of longer clips."""
    if not hasattr(transformers, "Qwen3OmniMoeThinkerForConditionalGeneration"):
        pytest.skip(f"transformers {transformers.__version__} has no Qwen3-Omni")
    torch.manual_seed(0)
    tc = dict(vocab_size=200, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=32, intermediate_size=256, moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
              norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], max_position_embeddings=512,
              rms_norm_eps=1e-5, rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True})
    vc = dict(depth=3, hidden_size=64, out_hidden_size=128, num_heads=4, intermediate_size=128, patch_size=4,
              spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=64,
              deepstack_visual_indexes=[0, 1])
    ac = dict(num_mel_bins=16, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, d_model=64,
              max_source_positions=100, n_window=50, output_dim=128, n_window_infer=200, conv_chunksize=3,
              downsample_hidden_size=8)
    AUD, AUD_START, AUD_END = 154, 155, 156
    hf_cfg = transformers.Qwen3OmniMoeThinkerConfig(
        text_config=tc, vision_config=vc, audio_config=ac, audio_token_id=AUD, audio_start_token_id=AUD_START,
        audio_end_token_id=AUD_END, position_id_per_seconds=25, **_TOK)
    hf_cfg._attn_implementation = "eager"
    hf = transformers.Qwen3OmniMoeThinkerForConditionalGeneration(hf_cfg).eval().float()
    _randomise(hf)
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = ["Qwen3OmniMoeThinkerForConditionalGeneration"], "float32"
    # the complete checkpoint nests the thinker's configuration
    cfg = ModelConfig.from_hf_config({"architectures": ["Qwen3OmniMoeForConditionalGeneration"], "thinker_config": d})
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=512, max_num_seqs=2, num_gpu_blocks=64)
    model = llm.engine.runner.model
    sd = {"thinker." + k: v for k, v in hf.state_dict().items()}
    with torch.inference_mode():
        loaded = model.load_weights(list(sd.items()))
    assert len(loaded) == len(sd)
    frames = 150                                                   # chunks of 100 and 50 frames -> 13 + 7 rows
    feats = torch.randn(frames, 16)
    with torch.no_grad():
        want_audio = hf.audio_tower(feats.T, feature_lens=torch.tensor([frames])).last_hidden_state.float()
    with torch.inference_mode():
        got_audio = model.audio_tower(feats, [frames]).float()
    assert model.audio_tower.output_lengths([frames]) == [20] and got_audio.shape == want_audio.shape
    assert (got_audio - want_audio).abs().max().item() < 1e-5
    img = hf_cfg.image_token_id
    px = torch.randn(1 * 4 * 6, 3 * 2 * 16)
    ids = [5, 6, AUD_START] + [AUD] * 20 + [AUD_END, 7, _TOK["vision_start_token_id"]] + [img] * 6 + \
          [_TOK["vision_end_token_id"], 8, 9]
    seq = torch.tensor([ids])
    with torch.no_grad():
        want = hf(input_ids=seq, input_features=feats.T[None], feature_attention_mask=torch.ones(1, frames, dtype=torch.long),
                  pixel_values=px, image_grid_thw=torch.tensor([[1, 4, 6]]), attention_mask=torch.ones_like(seq)).logits[0, -1].float()
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
                 multi_modal_data={"pixel_values": px, "image_grid_thw": [[1, 4, 6]], "input_features": feats,
                                   "feature_lens": [frames]})
    assert (seen[0][-1] - want).abs().max().item() < 1e-4
    # a three-frame video (2 s per temporal patch: positions 50 apart) and an image
    vid = hf_cfg.video_token_id
    pv = torch.randn(3 * 4 * 4, 3 * 2 * 16)
    ids = [5, 6, _TOK["vision_start_token_id"]] + [vid] * 12 + [_TOK["vision_end_token_id"], 7, 8,
           _TOK["vision_start_token_id"]] + [img] * 6 + [_TOK["vision_end_token_id"], 9]
    seq = torch.tensor([ids])
    with torch.no_grad():
        want = hf(input_ids=seq, pixel_values_videos=pv, video_grid_thw=torch.tensor([[3, 4, 4]]),
                  video_second_per_grid=torch.tensor([2.0]), pixel_values=px, image_grid_thw=torch.tensor([[1, 4, 6]]),
                  attention_mask=torch.ones_like(seq)).logits[0, -1].float()
    seen.clear()
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
                 multi_modal_data={"pixel_values": px, "image_grid_thw": [[1, 4, 6]], "pixel_values_videos": pv,
                                   "video_grid_thw": [[3, 4, 4]], "second_per_grid_ts": [2.0]})
    assert (seen[0][-1] - want).abs().max().item() < 1e-4


def test_gemma4_with_images_matches_the_transformers_implementation():
    """Gemma-4 vision tower (position rows looked up by x and y, 2-D rotary embedding, clipped linears, pooling,
    standardisation) on two images of different grids, and the logits after a prompt holding both: soft tokens after
    the embedding scale, per-layer inputs of placeholder rows from the padding token."""
    if not hasattr(transformers, "Gemma4ForConditionalGeneration"):
        pytest.skip(f"transformers {transformers.__version__} has no Gemma-4")
    torch.manual_seed(0)
    IMG, BOI, EOI = 150, 151, 152
    tc = dict(vocab_size=200, hidden_size=128, num_hidden_layers=4, layer_types=["sliding_attention", "full_attention"] * 2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=32, global_head_dim=32, intermediate_size=256,
              max_position_embeddings=256, sliding_window=8, hidden_size_per_layer_input=32,
              vocab_size_per_layer_input=200, num_kv_shared_layers=0)
    vc = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, patch_size=4, position_embedding_size=32, pooling_kernel_size=2, standardize=True,
              use_clipped_linears=True)
    hf_cfg = transformers.Gemma4Config(text_config=tc, vision_config=vc, audio_config=None, image_token_id=IMG,
                                       boi_token_id=BOI, eoi_token_id=EOI, video_token_id=153, audio_token_id=154)
    hf_cfg._attn_implementation = "eager"
    hf = transformers.Gemma4ForConditionalGeneration(hf_cfg).eval().float()
    _randomise(hf)
    with torch.no_grad():
        hf.model.vision_tower.std_bias.copy_(torch.randn(64) * 0.1)
        hf.model.vision_tower.std_scale.copy_(1 + 0.1 * torch.randn(64))
        for name, buf in hf.model.vision_tower.named_buffers():
            if name.endswith("_min"):
                buf.fill_(-0.8)
            elif name.endswith("_max"):
                buf.fill_(0.9)
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = ["Gemma4ForConditionalGeneration"], "float32"
    llm = LLM(ModelConfig.from_hf_config(d), device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=64)
    model = llm.engine.runner.model
    sd = hf.state_dict()
    with torch.inference_mode():
        loaded = model.load_weights(list(sd.items()))
    assert [k for k in sd if k not in loaded] == ["lm_head.weight"]         # tied to the embedding
    grids = [(1, 4, 6), (1, 6, 4)]
    px = torch.rand(sum(h * w for _, h, w in grids), 3 * 16)

    def positions(h, w):
        return torch.stack([torch.arange(w).repeat(h), torch.arange(h).repeat_interleave(w)], -1)

    # the reference takes one padded batch row per image: both images have 24 patches
    pos = torch.stack([positions(h, w) for _, h, w in grids])
    with torch.no_grad():
        want_v = hf.model.get_image_features(px.view(2, 24, -1), pos).pooler_output.float()
    with torch.inference_mode():
        got_v = model.embed_multimodal(px, grids).float()
    assert got_v.shape == (12, 128) and (got_v - want_v.reshape(12, 128)).abs().max().item() < 1e-4
    ids = [5, 6, BOI] + [IMG] * 6 + [EOI, 7, BOI] + [IMG] * 6 + [EOI, 8, 9]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=px.view(2, 24, -1), image_position_ids=pos).logits[0, -1].float()
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
                 multi_modal_data={"pixel_values": px, "image_grid_thw": [list(g) for g in grids]})
    assert (seen[0][-1] - want).abs().max().item() < 2e-4


@pytest.mark.parametrize("qk_norm,text_type,arch", [
    (False, "qwen2", "InternVLForConditionalGeneration"), (True, "qwen2", "InternVLForConditionalGeneration"),
    # Intern-S1 checkpoints use the same tensor layout over a Qwen3 decoder (q / k norms, no q/k/v biases)
    (True, "qwen3", "InternS1ForConditionalGeneration")], ids=["layernorm", "rmsnorm_qk_norm", "intern_s1_qwen3_decoder"])
def test_internvl_matches_the_transformers_implementation(qk_norm, text_type, arch):
    """InternVL in the transformers-native layout: InternViT tower (class token, position table, layer scale; the
    large towers' RMSNorm with q / k normalisation), pixel shuffle, projector; logits after a two-image prompt."""
    if not hasattr(transformers, "InternVLForConditionalGeneration"):
        pytest.skip(f"transformers {transformers.__version__} has no InternVL")
    torch.manual_seed(0)
    IMG = 150
    tc = dict(model_type=text_type, vocab_size=200, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, intermediate_size=256, max_position_embeddings=512, rms_norm_eps=1e-5)
    if text_type == "qwen3":
        tc["head_dim"] = 32
    vc = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, image_size=[32, 32],
              patch_size=[8, 8], num_channels=3, use_qk_norm=qk_norm, norm_type="rms_norm" if qk_norm else "layer_norm",
              attention_bias=qk_norm)
    hf_cfg = transformers.InternVLConfig(text_config=tc, vision_config=vc, image_token_id=IMG, downsample_ratio=0.5)
    hf_cfg._attn_implementation = "eager"
    hf = transformers.InternVLForConditionalGeneration(hf_cfg).eval().float()
    _randomise(hf)
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = [arch], "float32"
    llm = LLM(ModelConfig.from_hf_config(d), device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=32)
    model = llm.engine.runner.model
    sd = hf.state_dict()
    with torch.inference_mode():
        loaded = model.load_weights(list(sd.items()))
    assert [k for k in sd if k not in loaded] == ["lm_head.weight"]         # tied to the embedding
    images = torch.randn(2, 3, 32, 32)
    # patches row-major, each flattened as (channel, y, x)
    px = images.view(2, 3, 4, 8, 4, 8).permute(0, 2, 4, 1, 3, 5).reshape(2, 16, 3 * 64)
    with torch.no_grad():
        want_v = hf.model.get_image_features(images).pooler_output.float()
    with torch.inference_mode():
        got_v = model.embed_multimodal(px).float()
    assert got_v.shape == (8, 128) and (got_v - want_v.reshape(8, 128)).abs().max().item() < 1e-4
    ids = [5, 6] + [IMG] * 4 + [7, 8] + [IMG] * 4 + [9, 10, 11]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=images).logits[0, -1].float()
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True), multi_modal_data={"pixel_values": px})
    assert (seen[0][-1] - want).abs().max().item() < 1e-4


@pytest.mark.parametrize("moe", [False, True], ids=["dense", "moe"])
def test_qwen3_5_with_images_matches_the_transformers_implementation(moe):
    """Qwen3.5 / Qwen3.5-MoE with two images: Qwen3-VL tower in front of the hybrid decoder, interleaved M-RoPE on the
    rotated half of each head in the gated full-attention layers; logits after the prompt and four greedy tokens."""
    names = ("Qwen3_5MoeConfig", "Qwen3_5MoeForConditionalGeneration") if moe else ("Qwen3_5Config", "Qwen3_5ForConditionalGeneration")
    if not all(hasattr(transformers, n) for n in names):
        pytest.skip(f"transformers {transformers.__version__} has no {names[1]}")
    torch.manual_seed(0)
    tc = dict(Q35, vocab_size=200, max_position_embeddings=512,
              rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                               "mrope_section": [3, 3, 2], "mrope_interleaved": True})
    if moe:
        tc.update(moe_intermediate_size=64, shared_expert_intermediate_size=64, num_experts=4, num_experts_per_tok=2)
    vc = dict(depth=2, hidden_size=64, out_hidden_size=128, num_heads=4, intermediate_size=128, patch_size=4,
              spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=64,
              deepstack_visual_indexes=[])
    hf_cfg = getattr(transformers, names[0])(text_config=tc, vision_config=vc, **_TOK)
    hf_cfg._attn_implementation = "eager"
    hf = getattr(transformers, names[1])(hf_cfg).eval().float()
    _randomise(hf)
    d = hf_cfg.to_dict()
    d["architectures"], d["torch_dtype"] = [names[1]], "float32"
    llm = LLM(ModelConfig.from_hf_config(d), device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=32)
    model = llm.engine.runner.model
    with torch.inference_mode():
        loaded = model.load_weights(list(hf.state_dict().items()))
    assert len(loaded) == len(hf.state_dict())
    grids = [(1, 8, 12), (1, 4, 6)]
    px = torch.randn(sum(t * h * w for t, h, w in grids), 3 * 2 * 16)
    img = hf_cfg.image_token_id
    ids = [5, 6, 7] + [img] * 24 + [8, 9] + [img] * 6 + [10, 11, 12]
    gthw = torch.tensor(grids)
    seq, want, want_logits = torch.tensor([ids]), [], None
    for _ in range(4):
        with torch.no_grad():
            lg = hf(input_ids=seq, pixel_values=px, image_grid_thw=gthw, mm_token_type_ids=(seq == img).long()).logits[0, -1].float()
        want_logits = lg if want_logits is None else want_logits
        want.append(lg.argmax().item())
        seq = torch.cat([seq, torch.tensor([[want[-1]]])], 1)
    seen, compute_logits = [], model.compute_logits

    def recording(h):
        out = compute_logits(h)
        seen.append(out.detach().float().clone())
        return out

    model.compute_logits = recording
    out = llm.generate([ids], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True),
                       multi_modal_data={"pixel_values": px, "image_grid_thw": [list(g) for g in grids]})[0].token_ids
    assert (seen[0][-1] - want_logits).abs().max().item() < 2e-4
    assert out == want
