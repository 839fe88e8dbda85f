"""LoRA: op oracles, manager slotting, and engine output equal to a model with merged weights."""
import torch

from vllm_kunlun_b200 import LLM, SamplingParams
from vllm_kunlun_b200.config import llama_3_1_8b, tiny
from vllm_kunlun_b200.lora import LoRARequest, PunicaWrapperB200
from vllm_kunlun_b200.ops.reference import misc as ref


def _cfg(hidden=64, heads=4, kv=2, hd=16, inter=128, vocab=128):
    return tiny(llama_3_1_8b(), num_layers=2, vocab_size=vocab, hidden_size=hidden, num_heads=heads, num_kv_heads=kv,
                head_dim=hd, intermediate_size=inter, max_position=256, dtype="float32")


def _adapter(cfg, seed, r=4, alpha=8.0, targets=("q_proj", "v_proj", "o_proj", "gate_proj", "down_proj")):
    g = torch.Generator().manual_seed(seed)
    shapes = {"q_proj": (cfg.q_size, cfg.hidden_size), "k_proj": (cfg.kv_size, cfg.hidden_size),
              "v_proj": (cfg.kv_size, cfg.hidden_size), "o_proj": (cfg.hidden_size, cfg.q_size),
              "gate_proj": (cfg.intermediate_size, cfg.hidden_size), "up_proj": (cfg.intermediate_size, cfg.hidden_size),
              "down_proj": (cfg.hidden_size, cfg.intermediate_size)}
    t = {}
    for layer in range(cfg.num_layers):
        for name in targets:
            out_f, in_f = shapes[name]
            blk = "self_attn" if name in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{layer}.{blk}.{name}"
            t[f"{base}.lora_A.weight"] = torch.randn(r, in_f, generator=g) * 0.3
            t[f"{base}.lora_B.weight"] = torch.randn(out_f, r, generator=g) * 0.3
    return LoRARequest(f"a{seed}", seed, tensors=t, rank=r, alpha=alpha)


def test_segment_and_token_forms_agree():
    torch.manual_seed(0)
    x = torch.randn(10, 32)
    A, B = torch.randn(3, 4, 32), torch.randn(3, 16, 4)
    lod, ids = torch.tensor([0, 3, 3, 7, 10]), torch.tensor([1, 0, -1, 2])
    tok = PunicaWrapperB200.segments_to_token_ids(lod, ids)
    h1, h2 = ref.sgmv_shrink(x, A, lod, ids, 0.5), ref.bgmv_shrink(x, A, tok, 0.5)
    torch.testing.assert_close(h1, h2)
    o1 = ref.sgmv_expand(h1, B, lod, ids, torch.zeros(10, 20), offset=4)
    o2 = ref.bgmv_expand(h2, B, tok, torch.zeros(10, 20), offset=4)
    torch.testing.assert_close(o1, o2)
    assert o1[3:7].abs().sum() == 0 and o1[:, :4].abs().sum() == 0


def test_engine_with_adapters_matches_merged_weights():
    cfg = _cfg()
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    llm = LLM(cfg, enable_lora=True, max_loras=2, max_lora_rank=8, **kw)
    a1, a2 = _adapter(cfg, 1), _adapter(cfg, 2, r=8, alpha=4.0, targets=("k_proj", "up_proj", "o_proj"))
    prompts = [list(range(3, 20)), list(range(30, 41)), list(range(50, 58))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    mixed = [o.token_ids for o in llm.generate(prompts, sp, lora_request=[a1, a2, None])]

    def merged(adapter):
        m = LLM(cfg, **kw)
        if adapter is not None:
            sd = {}
            model = m.engine.runner.model
            base = {n: p for n, p in model.named_parameters()}
            scale = adapter.alpha / adapter.rank
            for layer in range(cfg.num_layers):
                qkv = base[f"layers.{layer}.self_attn.qkv_proj.weight"].data
                gu = base[f"layers.{layer}.mlp.gate_up_proj.weight"].data
                offs = {"q_proj": (qkv, 0), "k_proj": (qkv, cfg.q_size), "v_proj": (qkv, cfg.q_size + cfg.kv_size),
                        "gate_proj": (gu, 0), "up_proj": (gu, cfg.intermediate_size),
                        "o_proj": (base[f"layers.{layer}.self_attn.o_proj.weight"].data, 0),
                        "down_proj": (base[f"layers.{layer}.mlp.down_proj.weight"].data, 0)}
                for name, (w, off) in offs.items():
                    blk = "self_attn" if name in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
                    key = f"base_model.model.model.layers.{layer}.{blk}.{name}"
                    if f"{key}.lora_A.weight" in adapter.tensors:
                        d = adapter.tensors[f"{key}.lora_B.weight"] @ adapter.tensors[f"{key}.lora_A.weight"] * scale
                        with torch.inference_mode():
                            w[off:off + d.shape[0]] += d
        return m

    for i, ad in enumerate((a1, a2, None)):
        want = merged(ad).generate([prompts[i]], sp)[0].token_ids
        assert mixed[i] == want, (i, mixed[i], want)
    # a third adapter evicts the least recently used slot
    a3 = _adapter(cfg, 3)
    llm.add_lora(a3)
    mgr = llm.engine.runner.lora
    assert set(mgr.slot_of) == {2, 3} and mgr.slot_for(1) == -1
