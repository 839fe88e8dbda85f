"""Speculative decoding: the vectorised rejection sampler against the loop oracle, and MTP / n-gram
drafting through the engine (greedy outputs must equal plain decoding)."""
import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import RopeScaling, deepseek_v3, qwen2_0_5b, tiny
from vllm_kunlun_b200.ops.reference import misc as rx
from vllm_kunlun_b200.sample.rejection_sampler import RejectionSampler


@pytest.mark.parametrize("with_draft_probs", [False, True])
def test_rejection_sampler_matches_oracle(with_draft_probs):
    g = torch.Generator().manual_seed(0)
    B, V = 6, 50
    num_draft = torch.tensor([3, 0, 1, 4, 2, 4])
    n = int(num_draft.sum())
    tp = torch.rand(n, V, generator=g).softmax(-1)
    dp = torch.rand(n, V, generator=g).softmax(-1) if with_draft_probs else None
    draft = torch.randint(0, V, (n,), generator=g)
    # make some drafts match the target arg-max so greedy rows accept a few
    draft[0], draft[1] = tp[0].argmax(), tp[1].argmax()
    bonus = torch.randint(0, V, (B,), generator=g)
    is_greedy = torch.tensor([True, True, False, False, True, False])
    u = torch.rand(n, generator=g)
    q = torch.empty(B, V).exponential_(generator=g)
    cu = torch.zeros(B + 1, dtype=torch.long)
    cu[1:] = num_draft.cumsum(0)
    want = rx.rejection_sample(draft, cu, dp, tp, bonus, is_greedy, u, q, max_spec_len=4)
    got = RejectionSampler().forward(draft, num_draft, tp, bonus, is_greedy, dp, u, q, max_spec_len=4)
    assert torch.equal(got, want), (got, want)


def test_ngram_spec_decode_equals_plain():
    cfg = tiny(qwen2_0_5b(), num_layers=2, vocab_size=64, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=512)
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 64, (12,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, 64, (20,), generator=g).tolist()]
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    plain = LLM(cfg, device="cpu", block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64)
    spec = LLM(cfg, device="cpu", block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64,
               speculative_config={"method": "ngram", "num_speculative_tokens": 3})
    with torch.inference_mode():
        spec.engine.runner.model.load_state_dict(plain.engine.runner.model.state_dict())
    a = [o.token_ids for o in plain.generate(prompts, sp)]
    b = [o.token_ids for o in spec.generate(prompts, sp)]
    assert a == b
    assert spec.engine.stats["spec_proposed"] > 0


def test_mtp_spec_decode_equals_plain():
    cfg = tiny(deepseek_v3(fp8=False), num_layers=2, first_dense_layers=1, vocab_size=96, hidden_size=64, num_heads=2,
               num_kv_heads=2, q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=16,
               v_head_dim=16, head_dim=32, rotary_dim=16, intermediate_size=128, num_experts=4, num_experts_per_tok=2,
               moe_intermediate_size=64, n_group=2, topk_group=1, max_position=512, dtype="float32",
               rope_scaling=RopeScaling(), num_mtp_layers=1)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 96, (n,), generator=g).tolist() for n in (17, 40)]
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    plain = LLM(cfg, device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16)
    spec = LLM(cfg, device="cpu", block_size=64, max_model_len=256, max_num_seqs=4, num_gpu_blocks=16,
               speculative_config={"method": "mtp", "num_speculative_tokens": 1}, max_num_batched_tokens=32)
    with torch.inference_mode():
        spec.engine.runner.model.load_state_dict(plain.engine.runner.model.state_dict())
        spec.engine.runner.model.finish_loading()
    a = [o.token_ids for o in plain.generate(prompts, sp)]
    b = [o.token_ids for o in spec.generate(prompts, sp)]
    assert a == b  # verification makes the output independent of draft quality
    assert spec.engine.stats["spec_proposed"] > 0


@pytest.mark.parametrize("method", ["eagle", "eagle3"])
def test_eagle_drafts_do_not_change_greedy_output(method):
    """Whatever the (random-init) draft proposes, verification keeps the target's greedy tokens."""
    from vllm_kunlun_b200.config import llama_3_1_8b, tiny
    cfg = tiny(llama_3_1_8b(), num_layers=6, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=48)
    prompts = [list(range(3, 30)), list(range(40, 49))]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    want = [o.token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    llm = LLM(cfg, speculative_config={"method": method, "num_speculative_tokens": 1}, **kw)
    got = [o.token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    assert llm.engine.stats["spec_proposed"] > 0
    if method == "eagle3":
        assert llm.engine.runner.model.aux_hidden_state_layers == (2, 3, 3)
