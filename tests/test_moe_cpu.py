"""MoE routing / fused MoE oracles and the MoE engine path on CPU."""
import dataclasses

import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams, ops
from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
from vllm_kunlun_b200.ops.reference import basic as rb
from vllm_kunlun_b200.ops.reference import moe as rm


def test_routing_variants():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(7, 16, generator=g)
    w, ids = rm.route_softmax_topk(logits, 4, True)
    assert torch.allclose(w.sum(-1), torch.ones(7)) and ids.shape == (7, 4)
    p = logits.softmax(-1)
    assert torch.equal(ids.long(), p.topk(4).indices)
    bias = torch.randn(16, generator=g) * 0.1
    w2, ids2 = rm.route_sigmoid_group_topk(logits, bias, 4, n_group=4, topk_group=2, renormalize=True, scale=2.5)
    assert torch.allclose(w2.sum(-1), torch.full((7,), 2.5), atol=1e-5)
    # chosen experts come from at most topk_group groups
    assert all(len(set((ids2[t] // 4).tolist())) <= 2 for t in range(7))
    w3, ids3 = rm.route_topk_then_softmax(logits, 3)
    assert torch.allclose(w3.sum(-1), torch.ones(7))


def test_fused_moe_matches_dense_loop():
    g = torch.Generator().manual_seed(1)
    T, H, I, E, k = 9, 64, 32, 6, 2
    x = torch.randn(T, H, generator=g)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.1
    w2 = torch.randn(E, H, I, generator=g) * 0.1
    tw, ids = rm.route_softmax_topk(torch.randn(T, E, generator=g), k)
    out = rm.fused_moe(x, w13, w2, tw, ids)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            h = rb.silu_and_mul((x[t] @ w13[e].T).unsqueeze(0))
            ref[t] += tw[t, j] * (h @ w2[e].T).squeeze(0)
    assert torch.allclose(out, ref, atol=1e-4)
    # expert-parallel halves sum to the whole
    emap0 = torch.tensor([0, 1, 2, -1, -1, -1], dtype=torch.int32)
    emap1 = torch.tensor([-1, -1, -1, 0, 1, 2], dtype=torch.int32)
    a = rm.fused_moe(x, w13[:3], w2[:3], tw, ids, expert_map=emap0)
    b = rm.fused_moe(x, w13[3:], w2[3:], tw, ids, expert_map=emap1)
    assert torch.allclose(a + b, ref, atol=1e-4)


def test_fp8_block_quant_roundtrip_and_gemm():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(200, 384, generator=g) * 0.02
    q, s = rb.quant_fp8_block(w)
    assert s.shape == (2, 3)
    assert (rb.dequant_fp8_block(q, s) - w).abs().max() < 0.07 * w.abs().max()
    x = torch.randn(5, 384, generator=g)
    y = ops.fp8_linear(x, q, s, out_dtype=torch.float32)
    assert torch.allclose(y, x @ w.T, atol=0.05, rtol=0.1)


@pytest.mark.parametrize("fp8", [False, True])
def test_moe_engine_cpu(fp8):
    cfg = tiny(qwen3_30b_a3b(fp8=fp8), num_layers=2, vocab_size=256, hidden_size=128, num_heads=4, num_kv_heads=2,
               head_dim=32, intermediate_size=256, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
               max_position=512, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (12, 30)]
    a = llm.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))
    # chunked prefill must not change the result
    llm2 = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32,
               max_num_batched_tokens=16)
    with torch.inference_mode():
        llm2.engine.runner.model.load_state_dict(llm.engine.runner.model.state_dict())
    b = llm2.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))
    assert [o.token_ids for o in a] == [o.token_ids for o in b]


def test_int8_and_awq_expert_checkpoints_dequantise_on_load():
    """compressed-tensors W8A8 and AWQ-packed experts end up as the dense weights they encode."""
    import dataclasses

    from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
    from vllm_kunlun_b200.models.moe import FusedExperts
    from vllm_kunlun_b200.ops.reference import basic as rb
    base = tiny(qwen3_30b_a3b(fp8=False), num_layers=1, vocab_size=64, hidden_size=64, num_heads=2, num_kv_heads=1,
                head_dim=32, intermediate_size=64, num_experts=2, num_experts_per_tok=1, moe_intermediate_size=32,
                dtype="float32")
    g = torch.Generator().manual_seed(0)
    H, I = 64, 32
    # int8 per-channel
    ex = FusedExperts(dataclasses.replace(base, quantization="int8"), torch.float32, "cpu")
    want = {}
    for e in range(2):
        for which, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            w = torch.randn(*shape, generator=g)
            s = w.abs().amax(-1, keepdim=True) / 127
            q = torch.round(w / s).to(torch.int8)
            ex.load_expert(e, which, "weight", q)
            ex.load_expert(e, which, "weight_scale", s)
            want[(e, which)] = q.float() * s
    for e in range(2):
        torch.testing.assert_close(ex.w13.data[e, :I], want[(e, "gate_proj")])
        torch.testing.assert_close(ex.w13.data[e, I:], want[(e, "up_proj")])
        torch.testing.assert_close(ex.w2.data[e], want[(e, "down_proj")])
    # AWQ int4, group 32
    ex = FusedExperts(dataclasses.replace(base, quantization="awq"), torch.float32, "cpu")
    for which, (N, K) in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
        wi = torch.randint(0, 16, (K, N), generator=g)
        zi = torch.randint(0, 16, (K // 32, N), generator=g)
        sc = torch.rand(K // 32, N, generator=g) * 0.1
        qw, qz = rb.awq_pack(wi), rb.awq_pack(zi)
        for pname, t in (("qweight", qw), ("qzeros", qz), ("scales", sc)):
            ex.load_expert(1, which, pname, t)
        dense = rb.awq_dequantize(qw, sc, qz, 32).T
        got = ex.w2.data[1] if which == "down_proj" else ex.w13.data[1, (0 if which == "gate_proj" else I):][:I]
        torch.testing.assert_close(got, dense)
    # compressed-tensors W4A16 (pack-quantized, symmetric: values stored with an offset of 8), group 32
    ex = FusedExperts(dataclasses.replace(base, quantization="w4a16", quantization_kw={"group_size": 32, "symmetric": True}),
                      torch.float32, "cpu")
    for which, (N, K) in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
        qv = torch.randint(0, 16, (N, K), generator=g)
        sc = torch.rand(N, K // 32, generator=g) * 0.1
        wp = torch.zeros(N, K // 8, dtype=torch.int64)
        for j in range(8):
            wp |= qv[:, j::8].long() << (4 * j)
        wp = torch.where(wp >= 2 ** 31, wp - 2 ** 32, wp).to(torch.int32)
        for pname, t in (("weight_shape", torch.tensor([N, K])), ("weight_packed", wp), ("weight_scale", sc)):
            ex.load_expert(0, which, pname, t)
        dense = (qv.float() - 8) * sc.repeat_interleave(32, 1)
        got = ex.w2.data[0] if which == "down_proj" else ex.w13.data[0, (0 if which == "gate_proj" else I):][:I]
        torch.testing.assert_close(got, dense)
