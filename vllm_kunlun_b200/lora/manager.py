"""Adapter manager: owns the stacked A / B tensors of every LoRA-capable linear and the slot table.

The reference relies on upstream's LoRA model manager and only supplies the Punica wrapper through
``Platform.get_punica_wrapper`` (``platforms/kunlun.py:342-347``); this framework is standalone and carries
the manager as well.  Adapter checkpoints use PEFT naming
(``base_model.model.model.layers.N.self_attn.q_proj.lora_A.weight`` ``[r, in]``, ``...lora_B.weight`` ``[out, r]``).

Tensor-parallel layout: column-parallel linears keep ``A`` whole and shard ``B`` rows like the base weight;
row-parallel linears shard ``A`` columns and keep ``B`` whole - every rank then adds ``B (A_r x_r)`` to its
partial output and the layer's reduction sums the adapters together with the base GEMM."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..attention.metadata import get_forward_context
from ..models.layers import ColumnParallelLinear, RowParallelLinear
from .punica import PunicaWrapperB200

# checkpoint projection name -> (fused module name, slice index)
_PACKED = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
           "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}


@dataclass
class LoRARequest:
    lora_name: str
    lora_int_id: int
    lora_path: Optional[str] = None
    tensors: Optional[dict] = None  # in-memory adapter (tests, programmatic use)
    rank: Optional[int] = None
    alpha: Optional[float] = None


class _LoRAState:
    """Stacked adapters of one linear."""

    def __init__(self, mod, max_loras: int, max_rank: int, dtype, device):
        self.mod = mod
        if isinstance(mod, ColumnParallelLinear):
            self.slices = list(mod.local_sizes)
            k = mod.in_features
            self.a = [torch.zeros(max_loras, max_rank, k, dtype=dtype, device=device) for _ in self.slices]
            self.b = [torch.zeros(max_loras, n, max_rank, dtype=dtype, device=device) for n in self.slices]
        else:
            self.slices = [mod.out_features]
            self.a = [torch.zeros(max_loras, max_rank, mod.in_local, dtype=dtype, device=device)]
            self.b = [torch.zeros(max_loras, mod.out_features, max_rank, dtype=dtype, device=device)]

    def clear(self, slot: int):
        for t in self.a + self.b:
            t[slot].zero_()

    def set(self, slot: int, sl: int, A: torch.Tensor, B: torch.Tensor, scaling: float):
        mod, r = self.mod, A.shape[0]
        if isinstance(mod, ColumnParallelLinear):
            n = mod.local_sizes[sl]
            row0 = 0 if mod.replicate[sl] else mod.tp_rank * n
            self.a[sl][slot, :r].copy_(A)
            self.b[sl][slot, :, :r].copy_(B[row0:row0 + n] * scaling)
        else:
            c0 = mod.tp_rank * mod.in_local
            self.a[0][slot, :r].copy_(A[:, c0:c0 + mod.in_local])
            self.b[0][slot, :, :r].copy_(B * scaling)


class LoRAManager:
    def __init__(self, model: torch.nn.Module, max_loras: int, max_rank: int, max_tokens: int, max_batches: int,
                 device, dtype):
        self.model, self.max_loras, self.max_rank = model, max_loras, max_rank
        self.device, self.dtype = torch.device(device), dtype
        self.punica = PunicaWrapperB200(max_tokens, max_batches, device)
        self.states: dict = {}
        self.slot_of: dict = {}  # lora_int_id -> slot
        self.lru: list = []
        from ..models import dense as _dense
        _dense.ACT_FUSION[0] = False  # adapters add to the separate gate / up outputs
        for mod in model.modules():
            if isinstance(mod, _dense.GatedMLP):
                mod.set_act_fused(False)
        for name, mod in model.named_modules():
            if isinstance(mod, (ColumnParallelLinear, RowParallelLinear)) and getattr(mod, "weight", None) is not None \
                    and mod.weight.dim() == 2 and name.split(".")[-1] != "in_proj_ba":
                st = _LoRAState(mod, max_loras, max_rank, dtype, device)
                if isinstance(mod, RowParallelLinear):
                    mod.push_ok = False  # the adapter's delta is added after the GEMM, before the reduction
                self.states[name] = st
                self._wrap(mod, st)

    def _wrap(self, mod, st: _LoRAState):
        base = mod.forward

        def forward(x):
            y = base(x)
            punica = get_forward_context().lora
            if punica is None or punica.no_lora:
                return y
            return punica.add_lora_linear(y, x, st.a, st.b, 1.0, st.slices)
        mod.forward = forward

    # ---- adapters
    def slot_for(self, lora_int_id: int) -> int:
        return self.slot_of.get(lora_int_id, -1) if lora_int_id >= 0 else -1

    def add_adapter(self, req: LoRARequest) -> int:
        if req.lora_int_id in self.slot_of:
            return self.slot_of[req.lora_int_id]
        if len(self.slot_of) >= self.max_loras:
            victim = self.lru.pop(0)
            slot = self.slot_of.pop(victim)
        else:
            slot = next(i for i in range(self.max_loras) if i not in self.slot_of.values())
        tensors, rank, alpha = req.tensors, req.rank, req.alpha
        if tensors is None:
            tensors, rank, alpha = self._read(req.lora_path)
        for st in self.states.values():
            st.clear(slot)
        pairs: dict = {}
        for name, w in tensors.items():
            n = name.removeprefix("base_model.model.").removeprefix("model.")
            if ".lora_A" in n:
                pairs.setdefault(n.split(".lora_A")[0], {})["A"] = w
            elif ".lora_B" in n:
                pairs.setdefault(n.split(".lora_B")[0], {})["B"] = w
        for target, ab in pairs.items():
            if "A" not in ab or "B" not in ab:
                continue
            r = ab["A"].shape[0]
            if r > self.max_rank:
                raise ValueError(f"adapter rank {r} exceeds max_lora_rank {self.max_rank}")
            parts = target.split(".")
            fused, sl = _PACKED.get(parts[-1], (parts[-1], 0))
            key = ".".join(parts[:-1] + [fused])
            if key not in self.states:
                continue  # a layer of another pipeline stage, or an unsupported target
            scaling = float(alpha if alpha is not None else r) / float(rank or r)
            self.states[key].set(slot, sl, ab["A"].to(self.device, self.dtype), ab["B"].to(self.device, self.dtype), scaling)
        self.slot_of[req.lora_int_id] = slot
        self.lru.append(req.lora_int_id)
        return slot

    def remove_adapter(self, lora_int_id: int):
        slot = self.slot_of.pop(lora_int_id, None)
        if slot is not None:
            self.lru.remove(lora_int_id)
            for st in self.states.values():
                st.clear(slot)

    @staticmethod
    def _read(path: str):
        from ..models.loader import load_safetensors
        with open(os.path.join(path, "adapter_config.json")) as f:
            cfg = json.load(f)
        return dict(load_safetensors(path)), cfg.get("r"), cfg.get("lora_alpha")
