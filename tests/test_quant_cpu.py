"""Quantised linear methods on the CPU oracle path: int8 W8A8, AWQ and GPTQ int4, fp8 block-128 with TP sharding."""
import pytest
import torch

from vllm_kunlun_b200.models.layers import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from vllm_kunlun_b200.ops.reference import basic as rb


def test_int8_w8a8_linear_dynamic_and_static():
    torch.manual_seed(0)
    w = torch.randn(48, 64) * 0.1
    x = torch.randn(5, 64)
    lin = ReplicatedLinear(64, 48, dtype=torch.float32, device="cpu", quant="int8")
    lin.method.quantize_(lin, w)
    torch.testing.assert_close(lin(x), x @ w.T, atol=0.05, rtol=0.05)
    stat = ReplicatedLinear(64, 48, dtype=torch.float32, device="cpu", quant="int8", quant_kw={"static_input_scale": True})
    stat.method.quantize_(stat, w)
    stat.input_scale.data.fill_(float(x.abs().max()) / 127)
    torch.testing.assert_close(stat(x), x @ w.T, atol=0.08, rtol=0.08)


def test_awq_linear_unpacks_once_and_matches_dequantised_weight():
    torch.manual_seed(1)
    K, N, g = 128, 64, 32
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(0, 16, (K // g, N))
    sc = torch.rand(K // g, N) * 0.05
    lin = ReplicatedLinear(K, N, dtype=torch.float32, device="cpu", quant="awq", quant_kw={"group_size": g})
    lin.qweight.data.copy_(rb.awq_pack(wi))
    lin.qzeros.data.copy_(rb.awq_pack(zi))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    assert lin.qweight is None and lin.weight.shape == (N, K)
    dense = ((wi - zi.repeat_interleave(g, 0)).float() * sc.repeat_interleave(g, 0))  # [K, N]
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ dense, atol=1e-4, rtol=1e-4)


def test_gptq_linear_matches_dequantised_weight():
    torch.manual_seed(2)
    K, N, g = 128, 32, 64
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(1, 16, (K // g, N))  # stored minus one
    sc = torch.rand(K // g, N) * 0.05
    qw = torch.zeros(K // 8, N, dtype=torch.int64)
    for j in range(8):
        qw |= wi[j::8].long() << (4 * j)
    qz = torch.zeros(K // g, N // 8, dtype=torch.int64)
    for j in range(8):
        qz |= (zi[:, j::8].long() - 1) << (4 * j)
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    lin = ReplicatedLinear(K, N, dtype=torch.float32, device="cpu", quant="gptq", quant_kw={"group_size": g})
    lin.qweight.data.copy_(to32(qw))
    lin.qzeros.data.copy_(to32(qz))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    dense = (wi - zi.repeat_interleave(g, 0)).float() * sc.repeat_interleave(g, 0)
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ dense, atol=1e-4, rtol=1e-4)


def test_fp8_block_scales_shard_with_the_weight():
    """Row shards of a merged projection and column shards of a row-parallel layer take the matching scale blocks
    (ceil-division rule for partitions that are not multiples of 128)."""
    torch.manual_seed(3)
    K = 256
    parts = [256, 128]
    w = torch.randn(sum(parts), K) * 0.1
    q, s = rb.quant_fp8_block(w, (128, 128))
    deq = rb.dequant_fp8_block(q, s, (128, 128))
    x = torch.randn(4, K)
    outs = []
    for rank in range(2):
        lin = ColumnParallelLinear(K, parts, dtype=torch.float32, device="cpu", quant="fp8", tp_size=2, tp_rank=rank)
        off_w, off_s = 0, 0
        for i, n in enumerate(parts):
            lin.load("weight", q[off_w:off_w + n], i)
            lin.load("weight_scale_inv", s[off_s:off_s + n // 128], i)
            off_w, off_s = off_w + n, off_s + n // 128
        outs.append(lin(x))
    full = x @ deq.T
    got = torch.cat([outs[0][:, :128], outs[1][:, :128], outs[0][:, 128:], outs[1][:, 128:]], -1)
    torch.testing.assert_close(got, full, atol=0.2, rtol=0.1)
    row = [RowParallelLinear(K, 64, dtype=torch.float32, device="cpu", quant="fp8", tp_size=2, tp_rank=r, reduce_results=False)
           for r in range(2)]
    w2 = torch.randn(64, K) * 0.1
    q2, s2 = rb.quant_fp8_block(w2, (128, 128))
    acc = 0
    for r, lin in enumerate(row):
        lin.load("weight", q2)
        lin.load("weight_scale_inv", s2)
        acc = acc + lin(x[:, r * 128:(r + 1) * 128])
    torch.testing.assert_close(acc, x @ rb.dequant_fp8_block(q2, s2, (128, 128)).T, atol=0.2, rtol=0.1)


def test_w4_pack_roundtrip_and_pair_extraction_order():
    """The kernels' packed layout: unpack inverts pack, and the pair (2 j, 2 j + 1) of a word's eight k values is
    `(w >> 4 j) & 0x000F000F` (low half, high half) - the extraction the decode GEMM performs."""
    from vllm_kunlun_b200.quantization.int4 import pack_w4, unpack_w4
    torch.manual_seed(4)
    q = torch.randint(0, 16, (5, 64))
    packed = pack_w4(q)
    assert packed.shape == (5, 32) and packed.dtype == torch.uint8
    assert torch.equal(unpack_w4(packed), q.to(torch.int32))
    b = packed.view(5, 8, 4).long()
    words = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    for j in range(4):
        t = (words >> (4 * j)) & 0x000F000F
        assert torch.equal(t & 0xFFFF, q.view(5, 8, 8)[..., 2 * j].long())
        assert torch.equal(t >> 16, q.view(5, 8, 8)[..., 2 * j + 1].long())


@pytest.mark.parametrize("fmt,g", [("awq", 128), ("awq", 64), ("gptq", 128)])
def test_w4_linear_keeps_packed_weights(fmt, g):
    """bf16 AWQ / GPTQ layers with kernel-friendly shapes keep only the packed bytes (+ scale / zero per group) and
    give the result of the de-quantised weight; a GPTQ layer with a permuted g_idx falls back to a 16-bit weight."""
    torch.manual_seed(5)
    K, N = 256, 48 if fmt == "gptq" else 64
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(1, 16, (K // g, N))
    sc = (torch.rand(K // g, N) * 0.05 + 0.01).bfloat16()
    lin = ReplicatedLinear(K, N, dtype=torch.bfloat16, device="cpu", quant=fmt, quant_kw={"group_size": g})
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    if fmt == "awq":
        lin.qweight.data.copy_(rb.awq_pack(wi))
        lin.qzeros.data.copy_(rb.awq_pack(zi))
    else:
        qw = torch.zeros(K // 8, N, dtype=torch.int64)
        for j in range(8):
            qw |= wi[j::8].long() << (4 * j)
        qz = torch.zeros(K // g, N // 8, dtype=torch.int64)
        for j in range(8):
            qz |= (zi[:, j::8].long() - 1) << (4 * j)
        lin.qweight.data.copy_(to32(qw))
        lin.qzeros.data.copy_(to32(qz))
    lin.scales.data.copy_(sc)
    lin.method.process_weights_after_loading(lin)
    assert lin.weight is None and lin.w4_packed.shape == (N, K // 2) and lin.w4_scale.shape == (N, K // g)
    dense = ((wi - zi.repeat_interleave(g, 0)).float() * sc.float().repeat_interleave(g, 0)).bfloat16()   # [K, N]
    x = torch.randn(3, K).bfloat16()
    torch.testing.assert_close(lin(x).float(), (x.float() @ dense.float()).bfloat16().float(), atol=2e-2, rtol=2e-2)
    if fmt == "gptq":
        lin2 = ReplicatedLinear(K, N, dtype=torch.bfloat16, device="cpu", quant="gptq", quant_kw={"group_size": g})
        lin2.qweight.data.copy_(to32(qw)); lin2.qzeros.data.copy_(to32(qz)); lin2.scales.data.copy_(sc)
        lin2.g_idx.data.copy_(torch.arange(K, dtype=torch.int32).flip(0) // g)       # activation-order checkpoint
        lin2.method.process_weights_after_loading(lin2)
        assert lin2.weight is not None and lin2.weight.shape == (N, K)


def _awq_tensors(wi, zi, sc):
    return {"qweight": rb.awq_pack(wi), "qzeros": rb.awq_pack(zi), "scales": sc}


def _gptq_tensors(wi, zi, sc, g):
    K, N = wi.shape
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    qw = torch.zeros(K // 8, N, dtype=torch.int64)
    for j in range(8):
        qw |= wi[j::8].long() << (4 * j)
    qz = torch.zeros(K // g, N // 8, dtype=torch.int64)
    for j in range(8):
        qz |= (zi[:, j::8].long() - 1) << (4 * j)
    return {"qweight": to32(qw), "qzeros": to32(qz), "scales": sc, "g_idx": torch.arange(K, dtype=torch.int32) // g}


@pytest.mark.parametrize("fmt", ["awq", "gptq"])
def test_w4_checkpoints_shard_over_tensor_parallel_ranks(fmt):
    """AWQ / GPTQ tensors are input-major ([K, N / 8], [K / 8, N], [K / g, N]): a merged column-parallel layer takes
    its output partitions along dim 1 (per projection or from one fused tensor), a row-parallel layer its inputs
    along dim 0; both ranks together give the product with the de-quantised weight."""
    torch.manual_seed(7)
    K, parts, g = 256, [128, 64], 64
    N = sum(parts)
    wi = torch.randint(0, 16, (K, N))
    zi = torch.randint(1, 16, (K // g, N))
    sc = (torch.rand(K // g, N) * 0.05 + 0.01).bfloat16()
    dense = ((wi - zi.repeat_interleave(g, 0)).float() * sc.float().repeat_interleave(g, 0)).bfloat16().float()  # [K, N]
    mk = (lambda a, b, c: _awq_tensors(a, b, c)) if fmt == "awq" else (lambda a, b, c: _gptq_tensors(a, b, c, g))
    x = torch.randn(5, K).bfloat16()
    want = x.float() @ dense
    for fused in (False, True):
        outs = []
        for rank in range(2):
            lin = ColumnParallelLinear(K, parts, dtype=torch.bfloat16, device="cpu", quant=fmt, tp_size=2, tp_rank=rank,
                                       quant_kw={"group_size": g})
            if fused:
                for name, t in mk(wi, zi, sc).items():
                    lin.load(name, t)
            else:
                off = 0
                for i, n in enumerate(parts):
                    for name, t in mk(wi[:, off:off + n], zi[:, off:off + n], sc[:, off:off + n]).items():
                        lin.load(name, t, i)
                    off += n
            lin.method.process_weights_after_loading(lin)
            assert lin.weight is None and lin.w4_packed.shape == (N // 2, K // 2)
            outs.append(lin(x).float())
        # rank r holds the r-th half of every partition
        got = torch.cat([outs[0][:, :64], outs[1][:, :64], outs[0][:, 64:], outs[1][:, 64:]], 1)
        torch.testing.assert_close(got, want, atol=0.05, rtol=0.02)
    total = 0
    for rank in range(2):
        lin = RowParallelLinear(K, N, dtype=torch.bfloat16, device="cpu", quant=fmt, tp_size=2, tp_rank=rank,
                                reduce_results=False, quant_kw={"group_size": g})
        for name, t in mk(wi, zi, sc).items():
            lin.load(name, t)
        lin.method.process_weights_after_loading(lin)
        assert lin.w4_packed.shape == (N, K // 4)
        total = total + lin(x[:, rank * (K // 2):(rank + 1) * (K // 2)].contiguous()).float()
    torch.testing.assert_close(total, want, atol=0.08, rtol=0.02)


@pytest.mark.parametrize("symmetric", [True, False])
def test_compressed_tensors_w4a16_linear(symmetric):
    """compressed-tensors pack-quantized int4 (output-major tensors, eight values per word along k; symmetric values
    stored with an offset of 8, asymmetric with a packed zero point): replicated and column-parallel layers."""
    torch.manual_seed(8)
    K, N, g = 256, 64, 128
    q = torch.randint(0, 16, (N, K))
    z = torch.full((N, K // g), 8) if symmetric else torch.randint(0, 16, (N, K // g))
    sc = (torch.rand(N, K // g) * 0.05 + 0.01).bfloat16()
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    wp = torch.zeros(N, K // 8, dtype=torch.int64)
    for j in range(8):
        wp |= q[:, j::8].long() << (4 * j)
    zp = torch.zeros(N // 8, K // g, dtype=torch.int64)
    for j in range(8):
        zp |= z[j::8].long() << (4 * j)
    dense = ((q - z.repeat_interleave(g, 1)).float() * sc.float().repeat_interleave(g, 1)).bfloat16().float()   # [N, K]
    x = torch.randn(4, K).bfloat16()
    kw = {"group_size": g, "symmetric": symmetric}
    lin = ReplicatedLinear(K, N, dtype=torch.bfloat16, device="cpu", quant="w4a16", quant_kw=kw)
    lin.weight_packed.data.copy_(to32(wp)); lin.weight_scale.data.copy_(sc)
    if not symmetric:
        lin.weight_zero_point.data.copy_(to32(zp))
    lin.method.process_weights_after_loading(lin)
    assert lin.weight is None and lin.weight_packed is None and lin.w4_packed.shape == (N, K // 2)
    torch.testing.assert_close(lin(x).float(), x.float() @ dense.T, atol=0.05, rtol=0.02)
    outs = []
    for rank in range(2):
        col = ColumnParallelLinear(K, [32, 32], dtype=torch.bfloat16, device="cpu", quant="w4a16", tp_size=2, tp_rank=rank,
                                   quant_kw=kw)
        col.load("weight_packed", to32(wp)); col.load("weight_scale", sc)
        if not symmetric:
            col.load("weight_zero_point", to32(zp))
        col.method.process_weights_after_loading(col)
        outs.append(col(x).float())
    got = torch.cat([outs[0][:, :16], outs[1][:, :16], outs[0][:, 16:], outs[1][:, 16:]], 1)
    torch.testing.assert_close(got, x.float() @ dense.T, atol=0.05, rtol=0.02)


def test_quantization_config_sets_method_and_arguments():
    from vllm_kunlun_b200.config import ModelConfig
    base = {"architectures": ["LlamaForCausalLM"], "vocab_size": 128, "hidden_size": 64, "num_hidden_layers": 1,
            "num_attention_heads": 2, "intermediate_size": 128}
    c = ModelConfig.from_hf_config(dict(base, quantization_config={"quant_method": "awq", "q_group_size": 64, "w_bit": 4}))
    assert c.quantization == "awq" and c.quantization_kw == {"group_size": 64, "bits": 4}
    c = ModelConfig.from_hf_config(dict(base, quantization_config={"quant_method": "gptq", "group_size": 128, "bits": 4,
                                                                  "desc_act": True}))
    assert c.quantization == "gptq" and c.quantization_kw == {"group_size": 128, "bits": 4, "desc_act": True}
    ct = {"quant_method": "compressed-tensors", "config_groups": {"group_0": {"weights": {
        "num_bits": 4, "type": "int", "strategy": "group", "group_size": 128, "symmetric": True}}}}
    c = ModelConfig.from_hf_config(dict(base, quantization_config=ct))
    assert c.quantization == "w4a16" and c.quantization_kw == {"group_size": 128, "bits": 4, "symmetric": True}
    ct["config_groups"]["group_0"]["weights"]["num_bits"] = 8
    assert ModelConfig.from_hf_config(dict(base, quantization_config=ct)).quantization == "int8"


def test_awq_dense_model_loads_per_projection_tensors_and_matches_dequantised_model():
    """A whole decoder (merged qkv and gate/up projections, row-parallel o / down) from an AWQ checkpoint with one
    tensor triple per projection: logits equal those of the same model built from the de-quantised 16-bit weights."""
    from vllm_kunlun_b200.config import llama_3_1_8b, tiny
    from vllm_kunlun_b200.models import build_model
    torch.manual_seed(9)
    g = 64
    base = tiny(llama_3_1_8b(), num_layers=2, vocab_size=96, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32,
                intermediate_size=256, max_position=128, dtype="bfloat16")
    import dataclasses
    qcfg = dataclasses.replace(base, quantization="awq", quantization_kw={"group_size": g, "bits": 4})
    ref = build_model(base, device="cpu")
    qm = build_model(qcfg, device="cpu")
    dense_sd, q_sd = {}, {}
    for name, p in ref.state_dict().items():
        dense_sd[name] = torch.randn(p.shape).mul(0.05).to(p.dtype) if p.dtype.is_floating_point else p.clone()
    proj = {"self_attn.q_proj": (128, 128), "self_attn.k_proj": (64, 128), "self_attn.v_proj": (64, 128),
            "self_attn.o_proj": (128, 128), "mlp.gate_proj": (256, 128), "mlp.up_proj": (256, 128),
            "mlp.down_proj": (128, 256)}
    ckpt_dense, ckpt_q = [], []
    for name, t in dense_sd.items():
        if ".layers." in name and ("_proj" in name):
            continue                                   # projections are generated below, per checkpoint projection
        ckpt_dense.append((name, t)); ckpt_q.append((name, t))
    for layer in range(2):
        for pj, (N, K) in proj.items():
            wi = torch.randint(0, 16, (K, N))
            zi = torch.randint(0, 16, (K // g, N))
            sc = (torch.rand(K // g, N) * 0.02 + 0.005).bfloat16()
            w = ((wi - zi.repeat_interleave(g, 0)).float() * sc.float().repeat_interleave(g, 0)).bfloat16().T.contiguous()
            ckpt_dense.append((f"model.layers.{layer}.{pj}.weight", w))
            for k, t in _awq_tensors(wi, zi, sc).items():
                ckpt_q.append((f"model.layers.{layer}.{pj}.{k}", t))
    with torch.inference_mode():
        ref.load_weights(ckpt_dense)
        loaded = qm.load_weights(ckpt_q)
    assert any(n.endswith("q_proj.qweight") for n in loaded) and any(n.endswith("down_proj.scales") for n in loaded)
    attn = qm.layers["0"].self_attn
    assert attn.qkv_proj.weight is None and attn.qkv_proj.w4_packed.shape == (256, 64)
    # both models on the same step: a 17-token prompt, hidden states -> logits
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
    eng = LLM(base, device="cpu", block_size=16, max_model_len=64, max_num_seqs=2, num_gpu_blocks=16).engine
    eng.add_request(list(range(3, 20)), SamplingParams(max_tokens=1))
    md, ids, _ = eng.runner.prepare(eng.scheduler.schedule())
    res = []
    for m in (ref, qm):
        with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
            h, _ = m(ids)
            res.append(m.compute_logits(h).float())
    torch.testing.assert_close(res[1], res[0], atol=0.05, rtol=0.05)


def test_int8_checkpoints_shard_over_tensor_parallel_ranks():
    """compressed-tensors W8A8: merged column-parallel layers take rows of `weight` and `weight_scale` per partition;
    row-parallel layers take columns of `weight` and the whole per-channel `weight_scale`."""
    torch.manual_seed(10)
    K, parts = 64, [32, 16]
    N = sum(parts)
    w = torch.randn(N, K)
    s = w.abs().amax(1, keepdim=True) / 127
    q = (w / s).round().clamp(-127, 127).to(torch.int8)
    x = torch.randn(3, K)
    want = x @ (q.float() * s).T
    outs = []
    for rank in range(2):
        lin = ColumnParallelLinear(K, parts, dtype=torch.float32, device="cpu", quant="int8", tp_size=2, tp_rank=rank)
        lin.load("weight", q); lin.load("weight_scale", s)          # fused checkpoint tensors
        lin.method.process_weights_after_loading(lin)
        outs.append(lin(x))
    got = torch.cat([outs[0][:, :16], outs[1][:, :16], outs[0][:, 32 - 16:], outs[1][:, 16:]], 1)
    torch.testing.assert_close(got, want, atol=0.3, rtol=0.05)      # dynamic per-token activation quantisation
    total = 0
    for rank in range(2):
        lin = RowParallelLinear(K, N, dtype=torch.float32, device="cpu", quant="int8", tp_size=2, tp_rank=rank,
                                reduce_results=False)
        lin.load("weight", q); lin.load("weight_scale", s)
        lin.method.process_weights_after_loading(lin)
        total = total + lin(x[:, rank * 32:(rank + 1) * 32].contiguous())
    torch.testing.assert_close(total, want, atol=0.3, rtol=0.05)


def test_internvl_own_config_layout_parses_with_the_decoders_traits():
    """InternVL's own checkpoints name the decoder section ``llm_config``; q / k norms, biases and rope base follow
    the architecture named there, the tower's options (RMSNorm, q / k normalisation) come from ``vision_config``."""
    from vllm_kunlun_b200.config import ModelConfig
    d = dict(architectures=["InternVLChatModel"], downsample_ratio=0.5, torch_dtype="bfloat16",
             llm_config=dict(architectures=["Qwen3ForCausalLM"], vocab_size=1000, hidden_size=256, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512,
                             rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=4096, tie_word_embeddings=False),
             vision_config=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                                image_size=448, patch_size=14, qk_normalization=True, norm_type="rms_norm", qkv_bias=False))
    c = ModelConfig.from_hf_config(d)
    assert (c.architecture, c.vision["text_architecture"]) == ("InternVLChatModel", "Qwen3ForCausalLM")
    assert c.qk_norm and not c.qkv_bias and c.head_dim == 64 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.vision["qk_norm"] and c.vision["norm"] == "rmsnorm" and (c.vision["patch"], c.vision["image_size"]) == (14, 448)
    d["llm_config"] = dict(d["llm_config"], architectures=["Qwen2ForCausalLM"])
    c = ModelConfig.from_hf_config(d)
    assert c.qkv_bias and not c.qk_norm
