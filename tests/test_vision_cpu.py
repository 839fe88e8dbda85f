"""Vision-language wrappers on the CPU oracle path: tower shapes, image-row injection, M-RoPE, chunked prefill."""
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import qwen2_0_5b, tiny
from vllm_kunlun_b200.models.vision import get_mrope_positions

IMG = 127


def _qwen_vl():
    cfg = tiny(qwen2_0_5b(), num_layers=2, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=512, dtype="float32")
    cfg.architecture = "Qwen2_5_VLForConditionalGeneration"
    cfg.vision = dict(depth=2, hidden=32, heads=2, patch=2, temporal_patch=1, merge=2, intermediate=64, in_channels=3,
                      norm="rmsnorm", gated_mlp=True, image_token_id=IMG, text_architecture="Qwen2ForCausalLM")
    cfg.mrope_section = (4, 6, 6)
    return cfg


def _intern():
    cfg = tiny(qwen2_0_5b(), num_layers=2, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=512, dtype="float32")
    cfg.architecture = "InternVLChatModel"
    cfg.vision = dict(depth=2, hidden=32, heads=2, patch=2, intermediate=64, in_channels=3, norm="layernorm", act="gelu",
                      layer_scale=True, image_size=8, downsample=0.5, image_token_id=IMG,
                      text_architecture="Qwen2ForCausalLM")
    return cfg


def test_mrope_positions():
    ids = [1, 2, IMG, IMG, IMG, IMG, 3, 4]
    pos, delta = get_mrope_positions(ids, [(1, 4, 4)], IMG, 2)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:6].tolist() == [2, 2, 2, 2]          # temporal axis constant inside one image
    assert pos[1, 2:6].tolist() == [2, 2, 3, 3] and pos[2, 2:6].tolist() == [2, 3, 2, 3]
    assert pos[:, 6].tolist() == [4, 4, 4] and delta == 6 - 8


def test_mrope_positions_of_a_video():
    """Two temporal patches of 2 x 2 merged patches: frame-major order, the temporal axis steps by 1 per patch
    (Qwen2-VL) or by seconds-per-patch x tokens_per_second truncated (Qwen2.5-VL); text continues after the largest
    position used."""
    VID = IMG + 1
    ids = [1, IMG, IMG, 2] + [VID] * 8 + [3]
    pos, delta = get_mrope_positions(ids, [(1, 2, 4)], IMG, 2, VID, [(2, 4, 4)])
    assert pos[:, 1:3].tolist() == [[1, 1], [1, 1], [1, 2]] and pos[:, 3].tolist() == [3, 3, 3]
    assert pos[0, 4:12].tolist() == [4, 4, 4, 4, 5, 5, 5, 5]
    assert pos[1, 4:12].tolist() == [4, 4, 5, 5, 4, 4, 5, 5] and pos[2, 4:12].tolist() == [4, 5, 4, 5, 4, 5, 4, 5]
    assert pos[:, 12].tolist() == [6, 6, 6] and delta == 7 - 13
    pos, delta = get_mrope_positions(ids, [(1, 2, 4)], IMG, 2, VID, [(2, 4, 4)], [2.5 * 2])
    assert pos[0, 4:12].tolist() == [4, 4, 4, 4, 9, 9, 9, 9] and pos[:, 12].tolist() == [10, 10, 10] and delta == 11 - 13


def test_qwen_vl_generation_uses_the_image_and_survives_chunking():
    cfg = _qwen_vl()
    grid = [(1, 8, 4)]  # 32 patches -> 8 merged tokens
    px = torch.randn(32, 3 * 1 * 2 * 2, generator=torch.Generator().manual_seed(0))
    prompt = [5, 6, 7] + [IMG] * 8 + [9, 10, 11, 12]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    mm = {"pixel_values": px, "image_grid_thw": grid}
    whole = LLM(cfg, max_num_batched_tokens=64, **kw)
    a = whole.generate([prompt, [3, 4, 5, 6]], sp, multi_modal_data=[mm, None])
    chunked = LLM(cfg, max_num_batched_tokens=16, **kw)  # the image straddles two prefill chunks
    b = chunked.generate([prompt, [3, 4, 5, 6]], sp, multi_modal_data=[mm, None])
    assert [o.token_ids for o in a] == [o.token_ids for o in b]

    def logits(mm_data):
        from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
        eng = whole.engine
        eng.add_request(prompt, SamplingParams(max_tokens=1), multi_modal_data=mm_data)
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        ctx = ForwardContext(md, eng.runner.kv_caches, eng.pstate, extras=eng.runner._step_extras)
        with torch.inference_mode(), set_forward_context(ctx):
            h, _ = eng.runner.model(ids)
            out = eng.runner.model.compute_logits(h[-1:]).float()
        eng.run_until_done()
        return out

    l1, l2 = logits(mm), logits({"pixel_values": px * -3.0, "image_grid_thw": grid})
    assert (l1 - l2).abs().max() > 1e-4  # the image content reaches the logits
    emb = whole.engine.runner.model.embed_multimodal(px, grid)
    assert emb.shape == (8, cfg.hidden_size)


def test_internvl_tower_and_generation():
    cfg = _intern()
    px = torch.randn(2, 16, 3 * 2 * 2, generator=torch.Generator().manual_seed(1))  # 2 tiles, 4x4 patches each
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    emb = llm.engine.runner.model.embed_multimodal(px)
    assert emb.shape == (2 * 4, cfg.hidden_size)  # pixel shuffle: 16 -> 4 tokens per tile
    prompt = [5] + [IMG] * 8 + [9, 10]
    out = llm.generate([prompt], SamplingParams(max_tokens=4, ignore_eos=True), multi_modal_data={"pixel_values": px})
    assert len(out[0].token_ids) == 4


def _qwen3_vl_moe(arch="Qwen3VLMoeForConditionalGeneration"):
    from vllm_kunlun_b200.config import qwen3_30b_a3b
    cfg = tiny(qwen3_30b_a3b(fp8=False), num_layers=3, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1,
               head_dim=32, intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
               max_position=512, dtype="float32")
    cfg.architecture = arch
    cfg.vision = dict(depth=3, hidden=32, heads=2, patch=2, temporal_patch=1, merge=2, intermediate=64, in_channels=3,
                      norm="layernorm", image_token_id=IMG, audio_token_id=126, deepstack_indexes=[0, 1],
                      audio=dict(hidden=32, heads=2, intermediate=64, depth=2, n_mels=8, n_window=4, n_window_infer=16,
                                 downsample_hidden=4))
    cfg.mrope_section = (4, 6, 6)
    return cfg


def test_qwen3_vl_moe_deepstack_reaches_the_decoder():
    """Qwen3-VL-MoE: MoE decoder + tower whose intermediate (deep-stack) features are added after the first decoder
    layers; zeroing the deep-stack mergers must change the output, and chunked prefill must not."""
    cfg = _qwen3_vl_moe()
    grid = [(1, 8, 4)]
    px = torch.randn(32, 3 * 1 * 2 * 2, generator=torch.Generator().manual_seed(0))
    prompt = [5, 6, 7] + [IMG] * 8 + [9, 10, 11, 12]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    mm = {"pixel_values": px, "image_grid_thw": grid}
    llm = LLM(cfg, max_num_batched_tokens=64, **kw)
    model = llm.engine.runner.model
    assert type(model.language_model).__name__ == "MoEForCausalLM" and model.num_deepstack == 2
    emb = model.embed_multimodal(px, grid)
    assert emb.shape == (8, 3 * cfg.hidden_size)  # main + two deep-stack features per merged token
    a = llm.generate([prompt], sp, multi_modal_data=mm)[0].token_ids
    b = LLM(cfg, max_num_batched_tokens=8, **kw).generate([prompt], sp, multi_modal_data=mm)[0].token_ids
    assert a == b

    def last_hidden():
        from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
        eng = llm.engine
        eng.add_request(prompt, SamplingParams(max_tokens=1), multi_modal_data=mm)
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        ctx = ForwardContext(md, eng.runner.kv_caches, eng.pstate, extras=eng.runner._step_extras)
        with torch.inference_mode(), set_forward_context(ctx):
            h, _ = eng.runner.model(ids)
        eng.run_until_done()
        return h[-1].float().clone()
    h1 = last_hidden()
    for m in model.visual.ds_fc2:
        m.weight.data.zero_()
        m.bias.data.zero_()
    h2 = last_hidden()
    assert (h1 - h2).abs().max() > 1e-5


def test_qwen3_omni_thinker_takes_audio_and_images():
    cfg = _qwen3_vl_moe("Qwen3OmniMoeForConditionalGeneration")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    model = llm.engine.runner.model
    g = torch.Generator().manual_seed(2)
    # chunks of 2 * n_window = 8 frames, each shrunk 8x by the convolutions: 10 frames -> 1 + 1, 17 frames -> 1 + 1 + 1
    feats = torch.randn(17 + 10, 8, generator=g)
    assert model.audio_tower.output_lengths([17, 10]) == [3, 2]
    px = torch.randn(16, 3 * 1 * 2 * 2, generator=g)      # one 4x4-patch image -> 4 merged tokens
    AUD = 126
    prompt = [5] + [AUD] * 3 + [6] + [IMG] * 4 + [7] + [AUD] * 2 + [8, 9]
    mm = {"pixel_values": px, "image_grid_thw": [(1, 4, 4)], "input_features": feats, "feature_lens": [17, 10]}
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    out = llm.generate([prompt], sp, multi_modal_data=mm)[0]
    assert len(out.token_ids) == 4
    # the audio content reaches the output: other features, other embeddings (the random 0.02-scale convolution
    # weights are scaled up so that the signal is not lost under the position table)
    for w in (model.audio_tower.conv1_w, model.audio_tower.conv2_w, model.audio_tower.conv3_w):
        w.data.mul_(20.0)
    emb, rows, pos, delta = model.encode_multimodal_data(prompt, mm)
    assert rows == [5, 6, 7, 8, 1, 2, 3, 10, 11] and emb.shape == (9, 3 * cfg.hidden_size)     # images, then audio
    emb2, _, _, _ = model.encode_multimodal_data(prompt, dict(mm, input_features=feats * -2.0))
    assert (emb[4:7] - emb2[4:7]).abs().max() > 1e-5 and torch.equal(emb[:4], emb2[:4])
    # audio only
    out = llm.generate([[5] + [AUD] * 3 + [6, 7]], sp,
                       multi_modal_data={"input_features": feats[:17], "feature_lens": [17]})[0]
    assert len(out.token_ids) == 4
