"""Sparse-MoE decoders with GQA attention: Qwen3-MoE / Qwen2-MoE / Mixtral / GPT-OSS shapes.

Reference behaviour being replaced: ``UnquantizedFusedMoEMethod.apply_monolithic`` hands router
logits to ``KunlunOps.fused_moe`` (``ops/fused_moe/layer.py:36-81``, stage graph
``ops/_kunlun_ops.py:397-637``); with expert parallelism it runs a Python loop over local experts
with boolean masks on TP-replicated tokens and lets the layer's all-reduce combine the result
(``fused_moe_ep``, ``ops/_kunlun_ops.py:639-696``; note it ignores sigmoid / grouped routing there).

Parallel layouts here:
* TP experts (default): every rank holds all experts with the intermediate dim sharded.
* EP: every rank holds ``E / ep`` whole experts.  Tokens are replicated after attention, each rank
  computes its local experts for the tokens routed to them, and the partial outputs are summed by
  the all-reduce fused into the next norm - or, with mapped peer memory, tokens travel through the
  dispatch / combine kernels of :mod:`vllm_kunlun_b200.parallel.ep_a2a`.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from ..parallel.state import get_state
from .dense import STACKED, DenseDecoderLayer, DenseForCausalLM, GatedMLP
from .layers import ReplicatedLinear, param


class FusedExperts(nn.Module):
    """Stacked expert weights ``w13 [E_local, 2*I_local, H]`` and ``w2 [E_local, H, I_local]``."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        st = get_state()
        self.cfg = cfg
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.use_ep = st.ep_size > 1
        if self.use_ep:
            assert E % st.ep_size == 0
            self.num_local = E // st.ep_size
            self.first = st.ep_rank * self.num_local
            self.i_local = I
            self.i_rank, self.i_size = 0, 1
            emap = torch.full((E,), -1, dtype=torch.int32)
            emap[self.first:self.first + self.num_local] = torch.arange(self.num_local, dtype=torch.int32)
            self.register_buffer("expert_map", emap.to(device), persistent=False)
        else:
            self.num_local, self.first = E, 0
            self.i_local = I // st.tp_size
            self.i_rank, self.i_size = st.tp_rank, st.tp_size
            self.expert_map = None
        self.fp8 = cfg.quantization == "fp8"
        wdt = torch.float8_e4m3fn if self.fp8 else dtype
        self.w13 = param(self.num_local, 2 * self.i_local, H, dtype=wdt, device=device)
        self.w2 = param(self.num_local, H, self.i_local, dtype=wdt, device=device)
        self.block = tuple(cfg.weight_block_size)
        if self.fp8:
            bn, bk = self.block
            self.w13_scale = param(self.num_local, -(-2 * self.i_local // bn), -(-H // bk), dtype=torch.float32,
                                   device=device)
            self.w2_scale = param(self.num_local, -(-H // bn), -(-self.i_local // bk), dtype=torch.float32,
                                  device=device)
        else:
            self.w13_scale = self.w2_scale = None
        self.b13 = self.b2 = None
        if cfg.moe_bias:
            self.b13 = param(self.num_local, 2 * self.i_local, dtype=dtype, device=device)
            self.b2 = param(self.num_local, H, dtype=dtype, device=device)
        self.act = cfg.hidden_act

    def forward(self, x, topk_w, topk_ids):
        return ops.fused_moe(x, self.w13, self.w2, topk_w, topk_ids, self.act, self.b13, self.b2, self.w13_scale,
                             self.w2_scale, self.block, self.expert_map)

    # ---- int8 / int4 expert checkpoints (compressed-tensors W8A8 and W4A16 MoE, ``moe_wna16``, AWQ / GPTQ experts;
    # ``quantization/compressed_tensors/compressed_tensors_moe.py:111-360``, ``quantization/moe_wna16.py:242-289``):
    # the pieces of one projection are collected and de-quantised ONCE into the 16-bit grouped-GEMM layout (the
    # reference de-quantises int4 experts to dense weights on every call).
    _QUANT_PIECES = {"weight_scale": ("weight", "weight_scale"), "weight_packed": ("weight_packed", "weight_scale"),
                     "weight_zero_point": ("weight_packed", "weight_scale", "weight_zero_point"),
                     "qweight": ("qweight", "scales", "qzeros"), "scales": ("qweight", "scales", "qzeros"),
                     "qzeros": ("qweight", "scales", "qzeros")}

    def _load_quantised(self, e: int, which: str, pname: str, w: torch.Tensor) -> bool:
        """Returns True when ``pname`` belongs to an int8 / int4 format (and was consumed)."""
        q = self.cfg.quantization
        if q not in ("int8", "awq", "gptq", "wna16", "w4a16"):
            return False
        if pname in ("bias", "g_idx", "weight_shape", "input_scale"):
            return True  # not needed by the de-quantised layout
        pend = self.__dict__.setdefault("_pending", {})
        slot = pend.setdefault((e, which), {})
        slot[pname] = w
        from ..ops.reference import basic as rb
        dense = None
        if q == "int8" and "weight" in slot and "weight_scale" in slot:
            dense = slot["weight"].float() * slot["weight_scale"].float().reshape(-1, 1)
        elif q == "w4a16" and "weight_packed" in slot and "weight_scale" in slot and (
                self.cfg.quantization_kw.get("symmetric", True) or "weight_zero_point" in slot):
            # compressed-tensors pack-quantized int4: eight values per word along k; symmetric values carry an offset of 8
            wp, sc = slot["weight_packed"], slot["weight_scale"].float()
            shifts = torch.arange(0, 32, 4, dtype=torch.int32)
            qv = ((wp.unsqueeze(-1) >> shifts) & 0xF).reshape(wp.shape[0], -1).float()          # [N, K]
            g = qv.shape[1] // sc.shape[1]
            if "weight_zero_point" in slot:
                zp = slot["weight_zero_point"]
                z = ((zp.unsqueeze(1) >> shifts.view(1, -1, 1)) & 0xF).reshape(-1, zp.shape[1]).float()
            else:
                z = torch.full_like(sc, 8.0)
            dense = (qv - z.repeat_interleave(g, 1)) * sc.repeat_interleave(g, 1)
        elif q in ("awq", "gptq", "wna16") and all(k in slot for k in ("qweight", "scales", "qzeros")):
            g = slot["qweight"].shape[0] * (1 if q == "awq" else 8) // slot["scales"].shape[0]
            if q == "awq":
                dense = rb.awq_dequantize(slot["qweight"], slot["scales"], slot["qzeros"], g).T
            else:
                K = slot["qweight"].shape[0] * 8
                gidx = torch.arange(K, dtype=torch.int32) // g
                dense = rb.gptq_dequantize(slot["qweight"], slot["scales"], slot["qzeros"], gidx, 4).T
        if dense is not None:
            del pend[(e, which)]
            self.load_expert(e, which, "weight", dense.to(self.w13.dtype), _raw=True)
        return True

    # ---- checkpoint loading: ``experts.{e}.{gate,up,down}_proj.{weight,weight_scale_inv}`` ----
    def load_expert(self, e: int, which: str, pname: str, w: torch.Tensor, _raw: bool = False):
        le = e - self.first
        if not (0 <= le < self.num_local):
            return
        if not _raw and self._load_quantised(e, which, pname, w):
            return
        scale = pname == "weight_scale_inv"
        I = self.i_local
        if which in ("gate_proj", "up_proj", "w1", "w3"):
            dst = self.w13_scale if scale else self.w13
            div = self.block[0] if scale else 1
            off = 0 if which in ("gate_proj", "w1") else -(-I // div)
            n = -(-I // div)
            src0 = (self.i_rank * I) // div
            dst.data[le, off:off + n].copy_(w[src0:src0 + n])
        else:
            dst = self.w2_scale if scale else self.w2
            div = self.block[1] if scale else 1
            n = -(-I // div)
            src0 = (self.i_rank * I) // div
            dst.data[le].copy_(w[:, src0:src0 + n])


class SparseMoEBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, bias=cfg.moe_bias, dtype=dtype, device=device)
        self.e_score_correction_bias = (param(cfg.num_experts, dtype=torch.float32, device=device)
                                        if cfg.router_bias else None)
        self.experts = FusedExperts(cfg, dtype, device)
        self.shared_experts = None
        if cfg.num_shared_experts:
            self.shared_experts = GatedMLP(cfg.hidden_size,
                                           cfg.shared_intermediate_size or cfg.moe_intermediate_size * cfg.num_shared_experts,
                                           dtype, device, cfg.quantization, "silu", reduce_results=False)
        self.shared_expert_gate = (ReplicatedLinear(cfg.hidden_size, 1, dtype=dtype, device=device)
                                   if cfg.shared_expert_gate else None)

    def _a2a(self, x):
        """The dispatch / combine exchange, created on first use when enabled (expert-parallel CUDA runs only)."""
        from .. import envs
        st = get_state()
        if not (self.experts.use_ep and x.is_cuda and envs.B200_EP_A2A and x.dtype == torch.bfloat16):
            return None
        if getattr(st, "ep_a2a", None) is None:
            if st.tp_comm is None or st.ep_size != st.tp_size:
                return None
            from ..parallel.ep_a2a import EPAll2All
            cap = -(-envs.B200_EP_A2A_MAX_TOKENS // st.ep_size)
            st.ep_a2a = EPAll2All(st.tp_comm, cap, self.cfg.hidden_size, self.cfg.num_experts_per_tok, self.cfg.num_experts,
                                  fp8_payload=self.experts.fp8, spin_limit=envs.B200_SPIN_LIMIT)
        a2a = st.ep_a2a
        chunk = -(-x.shape[0] // st.ep_size)
        return a2a if (x.shape[0] >= st.ep_size and chunk <= a2a.cap) else None

    def _forward_a2a(self, x, a2a):
        """Sequence-parallel MoE: this rank routes and dispatches only its slice of the (replicated) tokens; the
        routed result goes into its rows of the partial output, and the reduction fused into the next norm - which
        the shared-expert partial needs anyway - completes the other ranks' rows."""
        cfg, st, ex = self.cfg, get_state(), self.experts
        T = x.shape[0]
        chunk = -(-T // st.ep_size)
        lo, hi = min(T, st.ep_rank * chunk), min(T, (st.ep_rank + 1) * chunk)
        xl = x[lo:hi]
        if hi > lo:
            w, ids = ops.moe_route(ops.router_gemm(xl, self.gate.weight, self.gate.bias), cfg.num_experts_per_tok, cfg.scoring_func, cfg.norm_topk_prob,
                                   self.e_score_correction_bias, cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor)
        else:
            w = torch.zeros(0, cfg.num_experts_per_tok, dtype=torch.float32, device=x.device)
            ids = torch.zeros(0, cfg.num_experts_per_tok, dtype=torch.int32, device=x.device)
        routed = a2a.moe(xl, ids, w, ex.w13, ex.w2, ex.act, ex.b13, ex.b2, ex.w13_scale, ex.w2_scale, bound=chunk)
        if self.shared_experts is not None:
            out = self.shared_experts(x)
            if self.shared_expert_gate is not None:
                out = out * torch.sigmoid(self.shared_expert_gate(x).float()).to(out.dtype)
        else:
            out = torch.zeros_like(x)
        out[lo:hi] += routed
        return out

    def forward(self, x):
        cfg = self.cfg
        a2a = self._a2a(x)
        if a2a is not None:
            return self._forward_a2a(x, a2a)
        w, ids = ops.router_and_route(x, self.gate.weight, self.gate.bias, cfg.num_experts_per_tok, cfg.scoring_func,
                                      cfg.norm_topk_prob, self.e_score_correction_bias, cfg.n_group, cfg.topk_group,
                                      cfg.routed_scaling_factor)
        out = self.experts(x, w, ids)
        if self.shared_experts is not None:
            sh = self.shared_experts(x)
            if self.shared_expert_gate is not None:
                sh = sh * torch.sigmoid(self.shared_expert_gate(x).float()).to(sh.dtype)
            st = get_state()
            if self.experts.use_ep and st.tp_size > 1:
                # routed part is complete per rank only after the EP sum; shared part is a TP partial:
                # both are partial sums over the same ranks, so they add before the fused reduction
                pass
            out = out + sh
        return out  # partial over TP / EP ranks; reduced by the next norm


class MoEDecoderLayer(DenseDecoderLayer):
    def build_mlp(self, cfg, layer_idx, dtype, device):
        if cfg.layer_is_moe(layer_idx):
            return SparseMoEBlock(cfg, dtype, device)
        return GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quantization, cfg.hidden_act,
                        cfg.mlp_bias, reduce_results=False)


class MoEForCausalLM(DenseForCausalLM):
    layer_cls = MoEDecoderLayer

    def init_random(self, seed: int = 0, std: float = 0.02):
        """fp8 checkpoints: draw N(0, std) in fp32 and quantise per 128x128 absmax block."""
        from ..quantization.fp8 import Fp8BlockLinearMethod
        g = torch.Generator(device=self.device).manual_seed(seed + 1000 * get_state().tp_rank)

        g_rep = torch.Generator(device=self.device).manual_seed(seed + 7)  # replicated parameters (router, ...)
        replicated = self.replicated_param_names()

        def draw(shape, gen=None):
            return torch.randn(shape, generator=gen or g, device=self.device, dtype=torch.float32) * std

        done = set()
        for mname, m in self.named_modules():
            if isinstance(getattr(m, "method", None), Fp8BlockLinearMethod):
                q, s = _quant_block_device(draw(m.weight.shape), m.method.block)
                m.weight.data.copy_(q)
                m.weight_scale_inv.data.copy_(s)
                done.update({f"{mname}.weight", f"{mname}.weight_scale_inv"})
            elif isinstance(m, FusedExperts) and m.fp8:
                for wn, sn in (("w13", "w13_scale"), ("w2", "w2_scale")):
                    wt = getattr(m, wn)
                    for e in range(wt.shape[0]):
                        q, s = _quant_block_device(draw(wt.shape[1:]), m.block)
                        wt.data[e].copy_(q)
                        getattr(m, sn).data[e].copy_(s)
                    done.update({f"{mname}.{wn}", f"{mname}.{sn}"})
        for name, p in self.named_parameters():
            if name in done or p.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                continue
            if name.endswith("layer_scalar"):
                p.data.fill_(1.0)
            elif name.endswith("norm.weight") or "layernorm.weight" in name:
                p.data.fill_(0.0 if self.cfg.gemma_norm else 1.0)
            elif name.endswith("e_score_correction_bias"):
                p.data.zero_()
            else:
                p.data.copy_(draw(p.shape, g_rep if name in replicated else None).to(p.dtype))
        self.finish_loading()

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        rest = []
        loaded = set()
        for name, w in weights:
            if ".mlp.experts." in name and ".shared" not in name:
                # model.layers.L.mlp.experts.E.{gate,up,down}_proj.{weight,weight_scale_inv}
                parts = name.removeprefix("model.").split(".")
                if parts[4] in ("gate_up_proj", "down_proj") and w.dim() == 3:
                    # stacked form (checkpoints saved by transformers 5: experts.gate_up_proj [E, 2 I, H] with the gate
                    # rows first, experts.down_proj [E, H, I])
                    li = parts[1]
                    if li in self.layers and isinstance(self.layers[li].mlp, SparseMoEBlock):
                        ex = self.layers[li].mlp.experts
                        for e in range(w.shape[0]):
                            if parts[4] == "down_proj":
                                ex.load_expert(e, "down_proj", "weight", w[e])
                            else:
                                half = w.shape[1] // 2
                                ex.load_expert(e, "gate_proj", "weight", w[e, :half])
                                ex.load_expert(e, "up_proj", "weight", w[e, half:])
                        loaded.add(name)
                    continue
                li, e, which, pname = parts[1], int(parts[4]), parts[5], parts[6]
                if li in self.layers and isinstance(self.layers[li].mlp, SparseMoEBlock):
                    self.layers[li].mlp.experts.load_expert(e, which, pname, w)
                    loaded.add(name)
                continue
            name = name.replace(".mlp.gate.e_score_correction_bias", ".mlp.e_score_correction_bias")
            name = name.replace(".block_sparse_moe.", ".mlp.")
            name = name.replace(".mlp.shared_expert.", ".mlp.shared_experts.")      # Qwen2-MoE spelling
            rest.append((name, w))
        loaded |= super().load_weights(rest)
        return loaded


def _quant_block_device(w: torch.Tensor, block=(128, 128)):
    """128x128 absmax e4m3 quantisation on the tensor's own device."""
    N, K = w.shape
    bn, bk = block
    Np, Kp = -(-N // bn) * bn, -(-K // bk) * bk
    wp = torch.zeros(Np, Kp, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w
    v = wp.reshape(Np // bn, bn, Kp // bk, bk)
    scale = v.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-10) / 448.0
    q = (v / scale).clamp(-448, 448).reshape(Np, Kp)[:N, :K].to(torch.float8_e4m3fn)
    return q, scale.reshape(Np // bn, Kp // bk)
