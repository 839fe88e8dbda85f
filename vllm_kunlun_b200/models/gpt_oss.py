"""GPT-OSS: attention sinks with alternating sliding-window layers, and MoE experts with biases and the
clamped ``swigluoai`` activation.

Reference: ``vllm_kunlun/models/gpt_oss.py`` (sinks + alternating window :48-136; MoE with bias + ``swigluoai``
:139-194, served there by a Python loop over experts, ``ops/_kunlun_ops.py:433-468``).  The decoder itself is the
generic sparse-MoE model; this file only adapts the checkpoint layout:

* ``mlp.experts.gate_up_proj [E, H, 2I]`` interleaves gate (even columns) and up (odd columns); the grouped GEMM
  wants ``[E, 2I, H]`` with the gate rows first,
* ``mlp.experts.down_proj [E, I, H]`` is input-major,
* the router is called ``mlp.router``, the per-head sink logits ``self_attn.sinks``.
"""
from __future__ import annotations

from typing import Iterable

import torch

from ..parallel.state import get_state
from .moe import MoEForCausalLM, SparseMoEBlock


class GptOssForCausalLM(MoEForCausalLM):
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        st = get_state()
        rest, loaded = [], set()
        for name, w in weights:
            n = name.removeprefix("model.")
            parts = n.split(".")
            layer = self.layers[parts[1]] if len(parts) > 3 and parts[0] == "layers" and parts[1] in self.layers else None
            if layer is not None and parts[2] == "mlp" and parts[3] == "experts" and isinstance(layer.mlp, SparseMoEBlock):
                ex = layer.mlp.experts
                I, lo = ex.i_local, ex.i_rank * ex.i_local
                sel = slice(ex.first, ex.first + ex.num_local)
                key = parts[4]
                if key == "gate_up_proj":
                    # the clamped SwiGLU of this family (``ops.act_and_mul(..., "swigluoai")``) reads its input as
                    # interleaved (gate_0, up_0, gate_1, up_1, ...), the checkpoint's own order: keep it, taking this
                    # rank's slice of the intermediate dimension pair by pair
                    gate, up = w[sel, :, 0::2], w[sel, :, 1::2]  # [E, H, I_total]
                    g, u = gate[:, :, lo:lo + I].transpose(1, 2), up[:, :, lo:lo + I].transpose(1, 2)   # [E, I, H]
                    ex.w13.data.copy_(torch.stack([g, u], 2).reshape(g.shape[0], 2 * I, -1))
                elif key == "gate_up_proj_bias":
                    g, u = w[sel, 0::2][:, lo:lo + I], w[sel, 1::2][:, lo:lo + I]
                    ex.b13.data.copy_(torch.stack([g, u], 2).reshape(g.shape[0], 2 * I))
                elif key == "down_proj":
                    ex.w2.data.copy_(w[sel, lo:lo + I, :].transpose(1, 2))
                elif key == "down_proj_bias":
                    # the bias is added once: by the rank holding the first slice of the intermediate dimension
                    ex.b2.data.copy_(w[sel] if ex.i_rank == 0 else torch.zeros_like(w[sel]))
                else:
                    continue
                loaded.add(name)
                continue
            if layer is not None and parts[2] == "self_attn" and parts[3] == "sinks":
                h = layer.self_attn.num_heads
                layer.self_attn.sinks.data.copy_(w[st.tp_rank * h:(st.tp_rank + 1) * h].float())
                loaded.add(name)
                continue
            rest.append((name.replace(".mlp.router.", ".mlp.gate."), w))
        return loaded | super().load_weights(rest)
