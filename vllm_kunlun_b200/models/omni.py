"""Qwen3-Omni "thinker": audio tower + vision tower + sparse-MoE decoder.

Reference: ``vllm_kunlun/models/qwen3_omni_moe_thinker.py`` (1 781 lines: audio encoder, Qwen3-VL style vision
tower with deep-stack features, M-RoPE decoder, processor glue).  Here the thinker reuses this package's pieces:
the vision tower and image-row injection of :mod:`.vision`, the MoE decoder of :mod:`.moe`, and an audio encoder
built from the same transformer block (bidirectional varlen attention per clip).

Audio path: log-mel frames ``[n_frames, n_mels]`` are stacked ``stride`` at a time (the strided convolution stem
written as a GEMM, like the vision patch embedding), get sinusoidal positions, run through the encoder blocks per
clip, and are projected to the decoder width; each output row replaces one ``audio_token_id`` placeholder of the
prompt.  Audio placeholders advance all three rotary axes together, like text.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from .layers import ReplicatedLinear
from .vision import Qwen3VLMoeForConditionalGeneration, VisionBlock, _Norm, get_mrope_positions


class AudioEncoder(nn.Module):
    def __init__(self, ac: dict, out_hidden: int, dtype, device):
        super().__init__()
        self.ac = ac
        h = ac["hidden"]
        self.stride = ac.get("stride", 8)
        self.n_mels = ac.get("n_mels", 128)
        self.stem = ReplicatedLinear(self.n_mels * self.stride, h, bias=True, dtype=dtype, device=device)
        blk = dict(hidden=h, heads=ac["heads"], intermediate=ac["intermediate"], norm="layernorm", act="gelu")
        self.blocks = nn.ModuleList([VisionBlock(blk, dtype, device) for _ in range(ac["depth"])])
        self.ln_post = _Norm(h, 1e-5, "layernorm", dtype, device)
        self.proj1 = ReplicatedLinear(h, h, bias=True, dtype=dtype, device=device)
        self.proj2 = ReplicatedLinear(h, out_hidden, bias=True, dtype=dtype, device=device)

    def output_lengths(self, feature_lens) -> list:
        return [max(1, -(-int(n) // self.stride)) for n in feature_lens]

    @staticmethod
    def _sinusoids(n: int, dim: int, device) -> torch.Tensor:
        inc = math.log(10000.0) / (dim // 2 - 1)
        inv = torch.exp(-inc * torch.arange(dim // 2, dtype=torch.float32, device=device))
        t = torch.arange(n, dtype=torch.float32, device=device)[:, None] * inv[None]
        return torch.cat([t.sin(), t.cos()], 1)

    def forward(self, features: torch.Tensor, feature_lens) -> torch.Tensor:
        """``features [sum(n_frames), n_mels]`` (clips concatenated) -> ``[sum(out_len), out_hidden]``."""
        dt = self.stem.weight.dtype
        rows, lens = [], self.output_lengths(feature_lens)
        o = 0
        for n, m in zip(feature_lens, lens):
            clip = features[o:o + int(n)]
            o += int(n)
            pad = m * self.stride - clip.shape[0]
            if pad:
                clip = torch.cat([clip, clip.new_zeros(pad, clip.shape[1])])
            x = self.stem(clip.reshape(m, self.stride * self.n_mels).to(dt))
            rows.append(x + self._sinusoids(m, x.shape[1], x.device).to(dt))
        x = torch.cat(rows)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        cu = cu.to(x.device)
        for blk in self.blocks:
            x = blk(x, cu)
        x = self.ln_post(x)
        return self.proj2(torch.nn.functional.gelu(self.proj1(x).float()).to(dt))


class Qwen3OmniMoeThinker(Qwen3VLMoeForConditionalGeneration):
    """``multi_modal_data`` keys: ``pixel_values`` + ``image_grid_thw`` (images / video frames), ``input_features`` +
    ``feature_lens`` (audio).  Either may be absent."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        super().__init__(cfg, device, dtype)
        ac = cfg.vision.get("audio") or dict(hidden=cfg.vision["hidden"], heads=cfg.vision["heads"],
                                              intermediate=cfg.vision["intermediate"], depth=2)
        self.audio_tower = AudioEncoder(ac, cfg.hidden_size, self.dtype, device)
        self.audio_token_id = cfg.vision.get("audio_token_id", cfg.vocab_size - 2)

    @torch.inference_mode()
    def encode_multimodal_data(self, token_ids, data: dict):
        """Embeddings and prompt rows of every placeholder (image and audio), in prompt order, plus M-RoPE positions."""
        H = self.cfg.hidden_size
        width = H * (1 + self.num_deepstack)
        grid = data.get("image_grid_thw")
        grid = [tuple(int(x) for x in g) for g in (grid.tolist() if hasattr(grid, "tolist") else grid)] if grid is not None else []
        img = aud = None
        if data.get("pixel_values") is not None:
            img = self.visual(data["pixel_values"].to(self.device), grid)
        if data.get("input_features") is not None:
            a = self.audio_tower(data["input_features"].to(self.device), list(data["feature_lens"]))
            aud = torch.cat([a, a.new_zeros(a.shape[0], width - H)], 1) if width > H else a  # no deep-stack part
        img_rows = [i for i, t in enumerate(token_ids) if t == self.image_token_id]
        aud_rows = [i for i, t in enumerate(token_ids) if t == self.audio_token_id]
        assert (img is None and not img_rows) or len(img_rows) == img.shape[0], "image placeholders vs embeddings"
        assert (aud is None and not aud_rows) or len(aud_rows) == aud.shape[0], "audio placeholders vs embeddings"
        parts = [(r, img[k]) for k, r in enumerate(img_rows)] if img is not None else []
        parts += [(r, aud[k]) for k, r in enumerate(aud_rows)] if aud is not None else []
        parts.sort(key=lambda p: p[0])
        rows = [r for r, _ in parts]
        embeds = torch.stack([e for _, e in parts]) if parts else torch.zeros(0, width, dtype=self.dtype, device=self.device)
        pos, delta = get_mrope_positions(token_ids, grid, self.image_token_id, self.visual.merge)
        return embeds, rows, pos, delta

    def init_random(self, seed: int = 0, std: float = 0.02):
        super().init_random(seed, std)
        g = torch.Generator(device=self.device).manual_seed(seed + 99)
        for name, p in self.audio_tower.named_parameters():
            if name.endswith("weight") and p.dim() == 1:
                p.data.fill_(1.0)
            elif name.endswith("bias"):
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g, device=self.device, dtype=torch.float32) * std).to(p.dtype))

    def load_weights(self, weights):
        aud = dict(self.audio_tower.named_parameters())
        rest, loaded = [], set()
        for name, w in weights:
            n = name.removeprefix("thinker.")
            if n.startswith("audio_tower."):
                k = n[len("audio_tower."):]
                if k in aud:
                    aud[k].data.copy_(w.reshape(aud[k].shape))
                    loaded.add(name)
                continue
            rest.append((n.replace("model.language_model.", "model.").replace("model.visual.", "visual."), w))
        return loaded | super().load_weights(rest)
