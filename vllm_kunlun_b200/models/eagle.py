"""EAGLE / EAGLE-3 draft models and the interfaces a target model offers them.

Reference: ``vllm_kunlun/models/interfaces.py`` (``EagleModelMixin``, ``SupportsEagle3``: the target exposes the
hidden states of a few chosen layers) and ``v1/sample/spec_decode/eagle.py:22-252`` (the proposer that drives
``eagle`` / ``eagle3`` / ``mtp`` drafts).

EAGLE: ``h0 = fc([embed(token_{i+1}) | target_hidden_i])`` -> a small stack of decoder layers -> the target's LM
head.  EAGLE-3: the target's auxiliary hidden states (low / middle / high layer) are first projected
``[3H] -> H`` and take the place of the last-layer hidden state; the draft has its own final norm."""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..parallel.state import get_state
from .dense import DenseDecoderLayer, DenseForCausalLM
from .layers import DTYPES, ParallelLMHead, RMSNorm, ReplicatedLinear, VocabParallelEmbedding


class EagleModelMixin:
    """Target-side half of EAGLE-3: remember which layers' outputs the draft wants."""

    aux_hidden_state_layers: tuple = ()

    def set_aux_hidden_state_layers(self, layers) -> None:
        self.aux_hidden_state_layers = tuple(layers)

    def get_eagle3_aux_hidden_state_layers(self) -> tuple:
        n = self.cfg.num_layers
        return (2, n // 2, n - 3) if n >= 6 else tuple(range(min(3, n)))


SupportsEagle3 = EagleModelMixin


class EagleDraftModel(nn.Module):
    def __init__(self, cfg: ModelConfig, device="cpu", dtype=None, target: Optional[DenseForCausalLM] = None,
                 num_layers: int = 1, eagle3: bool = False):
        super().__init__()
        self.cfg, self.eagle3 = cfg, eagle3
        self.dtype = dtype or DTYPES[cfg.dtype]
        self.device = torch.device(device)
        H = cfg.hidden_size
        self.first_layer = cfg.num_layers
        self.aux_proj = ReplicatedLinear(3 * H, H, dtype=self.dtype, device=device) if eagle3 else None
        self.fc = ReplicatedLinear(2 * H, H, dtype=self.dtype, device=device)
        self.layers = nn.ModuleDict({str(cfg.num_layers + i): DenseDecoderLayer(cfg, cfg.num_layers + i, self.dtype, device)
                                     for i in range(num_layers)})
        self.norm = RMSNorm(H, cfg.rms_norm_eps, self.dtype, device) if eagle3 else None
        if target is not None:
            self.embed_tokens, self.lm_head = target.embed_tokens, target.lm_head
        else:
            self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, H, self.dtype, device)
            self.lm_head = ParallelLMHead(cfg.vocab_size, H, self.dtype, device)

    def forward(self, input_ids, prev_hidden, step: int = 0):
        if self.aux_proj is not None:
            prev_hidden = self.aux_proj(prev_hidden)
        h = self.fc(torch.cat([self.embed_tokens(input_ids), prev_hidden], -1))
        residual, partial = None, False
        for layer in self.layers.values():
            h, residual = layer(h, residual, partial)
            partial = True
        st = get_state()
        if st.tp_size > 1:
            h = st.tp_comm.all_reduce(h)
        return h + residual

    def compute_logits(self, hidden, step: int = 0):
        return self.lm_head.logits(hidden if self.norm is None else self.norm(hidden))

    def kv_cache_spec(self, block_size: int):
        st = get_state()
        kvh = max(1, self.cfg.num_kv_heads // st.tp_size)
        return {int(k): ((2, kvh, block_size, self.cfg.head_dim), self.dtype) for k in self.layers}

    def init_random(self, seed: int = 0, std: float = 0.02):
        """Random draft weights; the embedding and LM head belong to the target and are left alone."""
        g = torch.Generator(device=self.device).manual_seed(seed + 177 + 1000 * get_state().tp_rank)
        g_rep = torch.Generator(device=self.device).manual_seed(seed + 178)
        replicated = self.replicated_param_names()
        for name, p in self.named_parameters():
            if name.startswith(("embed_tokens", "lm_head")) or not p.dtype.is_floating_point:
                continue
            if name.endswith("norm.weight") or "layernorm.weight" in name:
                p.data.fill_(1.0)
            else:
                gen = g_rep if name in replicated else g
                p.data.copy_((torch.randn(p.shape, generator=gen, device=self.device, dtype=torch.float32) * std).to(p.dtype))
        self.finish_loading()

    replicated_param_names = DenseForCausalLM.replicated_param_names
    finish_loading = DenseForCausalLM.finish_loading

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        """EAGLE checkpoints number their layers from 0 (``layers.0.*``, ``fc.weight``)."""
        off = self.first_layer
        renamed = []
        for name, w in weights:
            parts = name.removeprefix("model.").split(".")
            if parts[0] == "layers":
                parts[1] = str(int(parts[1]) + off)
            if parts[0] in ("embed_tokens", "lm_head"):
                continue
            renamed.append((".".join(parts), w))
        return DenseForCausalLM.load_weights(self, renamed)

    _resolve = DenseForCausalLM._resolve
    _attn_owner = DenseForCausalLM._attn_owner
