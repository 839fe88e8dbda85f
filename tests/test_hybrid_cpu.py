"""Qwen3-Next hybrid (gated delta net + gated attention + shared-expert MoE) on the CPU oracle path."""
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import qwen3_next_80b_a3b, tiny
from vllm_kunlun_b200.ops.reference import misc as ref


def _cfg():
    return tiny(qwen3_next_80b_a3b(), num_layers=4, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1,
                head_dim=32, rotary_dim=8, intermediate_size=128, num_experts=4, num_experts_per_tok=2,
                moe_intermediate_size=64, gdn_num_k_heads=2, gdn_num_v_heads=4, gdn_head_k_dim=16, gdn_head_v_dim=16,
                max_position=256, dtype="float32")


def test_chunked_and_recurrent_forms_agree():
    torch.manual_seed(0)
    L, Hk, Hv, Dk, Dv = 100, 2, 4, 16, 16
    q, k = torch.randn(L, Hk, Dk), torch.randn(L, Hk, Dk)
    v = torch.randn(L, Hv, Dv)
    g = -torch.rand(L, Hv)
    beta = torch.rand(L, Hv)
    S0 = torch.randn(Hv, Dv, Dk) * 0.1
    o1, s1 = ref.recurrent_gated_delta_rule(q, k, v, g, beta, S0)
    o2, s2 = ref.chunk_gated_delta_rule(q, k, v, g, beta, S0, chunk=32)
    torch.testing.assert_close(o1, o2, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(s1, s2, atol=2e-4, rtol=2e-4)


def test_hybrid_model_chunked_prefill_matches_whole_prefill():
    cfg = _cfg()
    prompts = [list(range(3, 45)), list(range(50, 61))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    whole = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32,
                max_num_batched_tokens=128)
    chunked = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32,
                  max_num_batched_tokens=16)
    a = [o.token_ids for o in whole.generate(prompts, sp)]
    b = [o.token_ids for o in chunked.generate(prompts, sp)]
    assert a == b
    # state slots are returned when requests finish
    assert len(whole.engine.scheduler.free_state_slots) == whole.engine.runner.num_state_slots


def test_hybrid_decode_consistent_with_prefill():
    """Tokens generated step by step (recurrent state) re-appear when the same text is scored as one prefill."""
    cfg = _cfg()
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    prompt = list(range(5, 25))
    out = llm.generate([prompt], SamplingParams(max_tokens=5, ignore_eos=True))[0].token_ids
    again = llm.generate([prompt + out[:4]], SamplingParams(max_tokens=1, ignore_eos=True))[0].token_ids
    assert again[0] == out[4]
