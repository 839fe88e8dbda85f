"""Engine on a B200: bf16 CUDA path vs the fp32 CPU oracle path, eager vs CUDA graph."""
import dataclasses

import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import llama_3_1_8b, tiny

pytestmark = pytest.mark.gpu


def _tiny():
    return tiny(llama_3_1_8b(), num_layers=2, vocab_size=2048, hidden_size=512, num_heads=8,
                               num_kv_heads=2, head_dim=64, intermediate_size=1024, max_position=4096)


def test_gpu_logits_match_cpu_oracle():
    cfg = _tiny()
    gpu = LLM(cfg, device="cuda", block_size=16, max_model_len=512, max_num_seqs=8, num_gpu_blocks=256,
              enforce_eager=True)
    cpu_cfg = dataclasses.replace(cfg, dtype="float32")
    cpu = LLM(cpu_cfg, device="cpu", block_size=16, max_model_len=512, max_num_seqs=8, num_gpu_blocks=256)
    sd = {k: v.float().cpu() for k, v in gpu.engine.runner.model.state_dict().items()}
    with torch.inference_mode():
        cpu.engine.runner.model.load_state_dict(sd)
    prompt = torch.randint(0, 2048, (150,), generator=torch.Generator().manual_seed(0)).tolist()

    def first_logits(llm):
        from vllm_kunlun_b200.engine.scheduler import ScheduledRequest, SchedulerOutput
        eng = llm.engine
        req = eng.add_request(prompt, SamplingParams(max_tokens=1))
        sched = eng.scheduler.schedule()
        md, ids, _ = eng.runner.prepare(sched)
        from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
        with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
            h, _ = eng.runner.model(ids)
            return eng.runner.model.compute_logits(h[-1:]).float().cpu()

    a, b = first_logits(gpu), first_logits(cpu)
    cos = torch.nn.functional.cosine_similarity(a, b).item()
    assert cos > 0.995, cos


def test_graph_decode_equals_eager():
    cfg = _tiny()
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (50, 9, 130)]
    outs = []
    for eager in (True, False):
        llm = LLM(cfg, device="cuda", block_size=16, max_model_len=512, max_num_seqs=8, num_gpu_blocks=256,
                  enforce_eager=eager, seed=3)
        outs.append([o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))])
        if not eager:
            assert llm.engine.runner.graphs.hits > 0
    assert outs[0] == outs[1]


def test_capture_all_then_generate_matches_lazy_capture():
    cfg = _tiny()
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (40, 12)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    kw = dict(device="cuda", block_size=16, max_model_len=512, max_num_seqs=8, num_gpu_blocks=256, seed=3)
    lazy = LLM(cfg, **kw)
    a = [o.token_ids for o in lazy.generate(prompts, sp)]
    warm = LLM(cfg, **kw)
    sizes = warm.engine.runner.graphs.capture_all()
    assert sizes and warm.engine.runner.profile_run(256) > 0
    b = [o.token_ids for o in warm.generate(prompts, sp)]
    assert a == b
