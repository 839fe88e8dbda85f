"""MiMo-V2-Flash: MoE decoder whose value heads are narrower than its query / key heads, with sliding-window
layers that carry a learned attention-sink bias.

Reference: ``vllm_kunlun/models/mimo_v2_flash.py`` (asymmetric ``v_head_dim`` QKV, SWA sink bias, V padded to
``head_dim`` before attention and sliced after :191-301; ``weight_scale_inv`` names :599) and the plugin's own
``QKVParallelLinear`` with a separate ``v_head_size`` (``ops/linear.py:427-782``).

Here the padding is moved into the weights at load time: the V rows of the fused QKV projection are laid out
``head_dim`` apart with zero rows in between, and ``o_proj`` gets matching zero columns.  The GEMMs then produce
/ consume the padded layout directly, the KV cache and both attention kernels see symmetric heads, and no
pad / slice kernels run per step.  fp8 block-quantised attention projections are de-quantised to bf16 when loaded
(their 128-row scale blocks do not survive the re-spacing); expert weights stay fp8.
"""
from __future__ import annotations

import dataclasses
from typing import Iterable

import torch

from ..config import ModelConfig
from .moe import MoEForCausalLM


def _dequant_block(w: torch.Tensor, s: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    bn, bk = block
    N, K = w.shape
    sf = s.float().repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
    return w.float() * sf


class MiMoV2FlashForCausalLM(MoEForCausalLM):
    def __init__(self, cfg: ModelConfig, device="cpu", dtype=None):
        self.ckpt_v_head_dim = cfg.v_head_dim
        self.attn_fp8 = cfg.quantization == "fp8" and cfg.v_head_dim != cfg.head_dim
        inner = dataclasses.replace(cfg, v_head_dim=cfg.head_dim,
                                    attn_quantization=None if self.attn_fp8 else cfg.attn_quantization)
        super().__init__(inner, device, dtype)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        cfg = self.cfg
        D, Dv, Hkv, H = cfg.head_dim, self.ckpt_v_head_dim, cfg.num_kv_heads, cfg.num_heads
        pending: dict = {}

        def fix(name, w):
            if Dv == D:
                return w
            if name.endswith("self_attn.v_proj.weight"):
                out = torch.zeros(Hkv, D, w.shape[-1], dtype=w.dtype)
                out[:, :Dv] = w.reshape(Hkv, Dv, -1)
                return out.reshape(Hkv * D, -1)
            if name.endswith("self_attn.v_proj.bias"):
                out = torch.zeros(Hkv, D, dtype=w.dtype)
                out[:, :Dv] = w.reshape(Hkv, Dv)
                return out.reshape(-1)
            if name.endswith("self_attn.o_proj.weight"):
                out = torch.zeros(w.shape[0], H, D, dtype=w.dtype)
                out[:, :, :Dv] = w.reshape(w.shape[0], H, Dv)
                return out.reshape(w.shape[0], H * D)
            return w

        def gen():
            for name, w in weights:
                if ".self_attn." in name and ("_proj.weight" in name) and Dv != D:
                    # pair fp8 weights with their block scales, hand on bf16
                    base = name.replace(".weight_scale_inv", ".weight")
                    slot = pending.setdefault(base, {})
                    slot["s" if name.endswith("weight_scale_inv") else "w"] = w
                    wq = slot.get("w")
                    if wq is not None and (wq.dtype != torch.float8_e4m3fn or "s" in slot):
                        full = _dequant_block(wq, slot["s"], cfg.weight_block_size).to(self.dtype) \
                            if wq.dtype == torch.float8_e4m3fn else wq
                        del pending[base]
                        yield base, fix(base, full)
                    continue
                if name.endswith("attention_sink_bias"):
                    name = name.replace("attention_sink_bias", "sinks")
                yield name, fix(name, w)
        return super().load_weights(gen())
