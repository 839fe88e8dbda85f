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


def test_batched_chunked_form_and_its_dispatch(monkeypatch):
    """The all-chunks-at-once form equals the token-by-token rule (length not a multiple of the chunk, grouped heads,
    an initial state); with ``B200_GDN_CHUNKED=1`` the varlen op sends long requests through it and the others through
    the recurrent pass, and leaves the same outputs and states as without the switch."""
    from vllm_kunlun_b200 import ops
    torch.manual_seed(1)
    L, Hk, Hv, Dk, Dv = 150, 2, 4, 16, 32
    q, k, v = torch.randn(L, Hk, Dk), torch.randn(L, Hk, Dk), torch.randn(L, Hv, Dv)
    g, beta = -torch.rand(L, Hv) * 0.5, torch.rand(L, Hv)
    S0 = torch.randn(Hv, Dv, Dk) * 0.1
    o1, s1 = ref.recurrent_gated_delta_rule(q, k, v, g, beta, S0)
    o2, s2 = ref.chunk_gated_delta_rule_batched(q, k, v, g, beta, S0, chunk=64)
    torch.testing.assert_close(o1, o2, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(s1, s2, atol=2e-4, rtol=2e-4)
    # three requests: 100 tokens with a state, 1 token (decode) with a state, 49 tokens without
    cu = torch.tensor([0, 100, 101, 150], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    has = torch.tensor([True, True, False])
    base = torch.randn(5, Hv, Dv, Dk) * 0.1

    def run():
        st = base.clone()
        return ops.gated_delta_rule(q, k, v, g, beta, st, cu, slots, has, None, True, cu.clone()), st

    calls, inner = [], ref.chunk_gated_delta_rule_batched
    monkeypatch.setattr(ref, "chunk_gated_delta_rule_batched", lambda *a, **kw: (calls.append(a[0].shape[0]), inner(*a, **kw))[1])
    monkeypatch.setenv("B200_GDN_CHUNKED", "0")
    want, want_st = run()
    assert calls == []
    monkeypatch.setenv("B200_GDN_CHUNKED", "1")
    got, got_st = run()
    assert calls == [100]                   # only the 100-token request took the chunked form
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(got_st, want_st, atol=2e-4, rtol=2e-4)
    assert torch.equal(got_st[1], base[1]) and torch.equal(got_st[4], base[4])      # untouched slots
    # and the model: same tokens either way
    cfg = _cfg()
    prompts = [list(range(3, 100)), list(range(50, 61))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(device="cpu", block_size=16, max_model_len=160, max_num_seqs=4, num_gpu_blocks=48, max_num_batched_tokens=160)
    b = [o.token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    monkeypatch.setenv("B200_GDN_CHUNKED", "0")
    a = [o.token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    assert a == b
