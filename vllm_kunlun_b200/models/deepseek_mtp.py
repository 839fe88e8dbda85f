"""DeepSeek multi-token-prediction (MTP) draft model.

Reference: ``vllm_kunlun/models/deepseek_mtp.py`` - one MTP layer = ``enorm`` / ``hnorm`` / ``eh_proj`` +
one decoder block + shared head (``:43-93``), multi-layer predictor (``:96-150``), checkpoint names
``model.layers.{num_layers + i}.*`` rewritten to the block (``:276-306``).

``forward(input_ids, prev_hidden)``: ``h = eh_proj([enorm(embed(ids)) | hnorm(prev_hidden)])`` then the
decoder block; position-0 embeddings are zeroed as in the reference (``:79-87``)."""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..parallel.state import get_state
from .deepseek import DeepseekDecoderLayer
from .layers import (DTYPES, ParallelLMHead, RMSNorm, ReplicatedLinear, VocabParallelEmbedding,
                     reduce_add_rmsnorm)


class MTPLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        H = cfg.hidden_size
        self.enorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.hnorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.eh_proj = ReplicatedLinear(2 * H, H, dtype=dtype, device=device)
        self.mtp_block = DeepseekDecoderLayer(cfg, layer_idx, dtype, device)
        self.shared_head_norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)

    def forward(self, embeds, prev_hidden, positions):
        # one kernel: position-0 mask, both RMSNorms and the concatenation
        x = ops.mtp_concat_norm(embeds, prev_hidden, self.enorm.weight, self.hnorm.weight, self.enorm.eps, positions)
        h = self.eh_proj(x)
        h, res = self.mtp_block(h, None, False)
        st = get_state()
        if st.tp_size > 1:
            h = st.tp_comm.all_reduce(h)
        return h + res


class DeepSeekMTP(nn.Module):
    """Draft model; shares the embedding and LM head tensors of the target when given."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=None, target=None):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype or DTYPES[cfg.dtype]
        self.device = torch.device(device)
        n = max(1, cfg.num_mtp_layers)
        self.first_layer = cfg.num_layers
        self.layers = nn.ModuleDict({str(cfg.num_layers + i): MTPLayer(cfg, cfg.num_layers + i, self.dtype, device)
                                     for i in range(n)})
        if target is not None:
            self.embed_tokens, self.lm_head = target.embed_tokens, target.lm_head
        else:
            self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, self.dtype, device)
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, self.dtype, device)

    def forward(self, input_ids, prev_hidden, step: int = 0):
        md = get_forward_context().attn
        layer = self.layers[str(self.first_layer + step % len(self.layers))]
        return layer(self.embed_tokens(input_ids), prev_hidden, md.positions)

    def compute_logits(self, hidden, step: int = 0):
        layer = self.layers[str(self.first_layer + step % len(self.layers))]
        return self.lm_head.logits(layer.shared_head_norm(hidden))

    def kv_cache_spec(self, block_size: int):
        cfg = self.cfg
        out = {}
        for k in self.layers:
            main = ((block_size, cfg.mla_cache_dim), self.dtype)
            out[int(k)] = [main, ((block_size, 132), torch.uint8)] if cfg.index_topk else main
        return out

    def init_random(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device=self.device).manual_seed(seed + 77)
        for name, p in self.named_parameters():
            if name.startswith(("embed_tokens", "lm_head")):
                continue
            if p.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                continue
            if "norm.weight" in name or "layernorm.weight" in name:
                p.data.fill_(1.0)
            elif name.endswith("e_score_correction_bias"):
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g, device=self.device, dtype=torch.float32) * std).to(p.dtype))
        self.finish_loading()

    def finish_loading(self):
        from .deepseek import MLAAttention
        for m in self.modules():
            meth = getattr(m, "method", None)
            if meth is not None:
                meth.process_weights_after_loading(m)
            if isinstance(m, MLAAttention):
                m.finish()

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        """``model.layers.{L}.{enorm,hnorm,eh_proj,shared_head.norm}`` stay on the MTP layer; every other
        tensor of layer ``L`` belongs to its decoder block (``.mtp_block.``)."""
        loaded = set()
        special = ("enorm", "hnorm", "eh_proj", "shared_head", "embed_tokens")
        for name, w in weights:
            parts = name.removeprefix("model.").split(".")
            if len(parts) < 3 or parts[0] != "layers" or parts[1] not in self.layers:
                continue
            layer = self.layers[parts[1]]
            rest = parts[2:]
            if rest[0] == "shared_head" and rest[1] == "norm":
                layer.shared_head_norm.weight.data.copy_(w)
            elif rest[0] in ("enorm", "hnorm"):
                getattr(layer, rest[0]).weight.data.copy_(w)
            elif rest[0] == "eh_proj":
                layer.eh_proj.weight.data.copy_(w)
            elif rest[0] in special:
                continue  # embedding / head are shared with the target
            else:
                continue  # decoder-block tensors are loaded through the target-style loader by the caller
            loaded.add(name)
        return loaded
