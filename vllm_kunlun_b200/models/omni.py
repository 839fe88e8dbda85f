"""Qwen3-Omni "thinker": audio tower + vision tower + sparse-MoE decoder.

Reference: ``vllm_kunlun/models/qwen3_omni_moe_thinker.py`` (1 781 lines: audio encoder, Qwen3-VL style vision
tower with deep-stack features, M-RoPE decoder, processor glue).  Here the thinker reuses this package's pieces:
the vision tower and image-row injection of :mod:`.vision`, the MoE decoder of :mod:`.moe`, and an audio encoder
built from the same transformer block (bidirectional varlen attention per window).

Audio path: a clip's log-mel frames ``[n_frames, n_mels]`` are cut into chunks of ``2 * n_window`` frames; each
chunk is an image ``[1, n_mels, frames]`` that three stride-2 3x3 convolutions (GELU after each) shrink 8x in both
directions; the (channel, mel) columns of every remaining time step are projected to the encoder width and get
sinusoidal positions counted from the start of their chunk; the valid time steps of a clip, concatenated, run through
the encoder blocks with attention inside windows of ``n_window_infer / (2 * n_window)`` chunks; LayerNorm and a
two-layer GELU projection map them to the decoder width.  Each output row replaces one ``audio_token_id``
placeholder of the prompt.  Audio placeholders advance all three rotary axes together, like text.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from .layers import ReplicatedLinear, param
from .vision import Qwen3VLMoeForConditionalGeneration, VisionBlock, _Norm


class AudioEncoder(nn.Module):
    def __init__(self, ac: dict, out_hidden: int, dtype, device):
        super().__init__()
        self.ac = ac
        h, c = ac["hidden"], ac.get("downsample_hidden", 480)
        self.n_mels = ac.get("n_mels", 128)
        self.n_window, self.n_window_infer = ac.get("n_window", 50), ac.get("n_window_infer", 400)
        self.conv_chunk = ac.get("conv_chunksize", 500)
        self.conv1_w, self.conv1_b = param(c, 1, 3, 3, dtype=dtype, device=device), param(c, dtype=dtype, device=device)
        self.conv2_w, self.conv2_b = param(c, c, 3, 3, dtype=dtype, device=device), param(c, dtype=dtype, device=device)
        self.conv3_w, self.conv3_b = param(c, c, 3, 3, dtype=dtype, device=device), param(c, dtype=dtype, device=device)
        self.conv_out = ReplicatedLinear(c * self._shrink(self.n_mels), h, bias=False, dtype=dtype, device=device)
        blk = dict(hidden=h, heads=ac["heads"], intermediate=ac["intermediate"], norm="layernorm", act="gelu", eps=1e-5)
        self.blocks = nn.ModuleList([VisionBlock(blk, dtype, device) for _ in range(ac["depth"])])
        self.ln_post = _Norm(h, 1e-5, "layernorm", dtype, device)
        self.proj1 = ReplicatedLinear(h, h, bias=True, dtype=dtype, device=device)
        self.proj2 = ReplicatedLinear(h, out_hidden, bias=True, dtype=dtype, device=device)

    @staticmethod
    def _shrink(n: int) -> int:
        """Length after the three stride-2, padding-1, 3-wide convolutions."""
        for _ in range(3):
            n = (n - 1) // 2 + 1
        return n

    def _chunks(self, n: int) -> list:
        win = 2 * self.n_window
        return [win] * (n // win) + ([n % win] if n % win else [])

    def output_lengths(self, feature_lens) -> list:
        """Audio tokens per clip: every chunk of ``2 * n_window`` frames (the tail may be shorter) shrinks 8x."""
        return [sum(self._shrink(c) for c in self._chunks(int(n))) for n in feature_lens]

    @staticmethod
    def _sinusoids(n: int, dim: int, device) -> torch.Tensor:
        inc = math.log(10000.0) / (dim // 2 - 1)
        inv = torch.exp(-inc * torch.arange(dim // 2, dtype=torch.float32, device=device))
        t = torch.arange(n, dtype=torch.float32, device=device)[:, None] * inv[None]
        return torch.cat([t.sin(), t.cos()], 1)

    def forward(self, features: torch.Tensor, feature_lens) -> torch.Tensor:
        """``features [sum(n_frames), n_mels]`` (clips concatenated) -> ``[sum(output_lengths), out_hidden]``."""
        dt = self.conv_out.weight.dtype
        lens = [c for n in feature_lens for c in self._chunks(int(n))]
        # chunks side by side, zero-padded on the right to the longest one (the convolutions see the padding of a
        # shorter tail chunk exactly as the released model does)
        T = max(lens)
        x = features.new_zeros(len(lens), 1, self.n_mels, T, dtype=dt)
        o = 0
        for i, n in enumerate(lens):
            x[i, 0, :, :n] = features[o:o + n].T.to(dt)
            o += n
        ys = []
        for part in x.split(self.conv_chunk):
            y = F.gelu(F.conv2d(part, self.conv1_w, self.conv1_b, stride=2, padding=1))
            y = F.gelu(F.conv2d(y, self.conv2_w, self.conv2_b, stride=2, padding=1))
            ys.append(F.gelu(F.conv2d(y, self.conv3_w, self.conv3_b, stride=2, padding=1)))
        y = torch.cat(ys)                                                   # [chunks, c, mel', t']
        b, c, f, t = y.shape
        y = self.conv_out(y.permute(0, 3, 1, 2).reshape(b * t, c * f)).view(b, t, -1)
        y = y + self._sinusoids(t, y.shape[-1], y.device).to(dt)
        x = torch.cat([y[i, :self._shrink(n)] for i, n in enumerate(lens)])
        window = t * max(1, self.n_window_infer // (2 * self.n_window))
        cu = [0]
        for total in self.output_lengths(feature_lens):
            for w in [window] * (total // window) + ([total % window] if total % window else []):
                cu.append(cu[-1] + w)
        cu = torch.tensor(cu, dtype=torch.int32).to(x.device)
        for blk in self.blocks:
            x = blk(x, cu)
        x = self.ln_post(x)
        return self.proj2(F.gelu(self.proj1(x).float()).to(dt))


class Qwen3OmniMoeThinker(Qwen3VLMoeForConditionalGeneration):
    """``multi_modal_data`` keys: ``pixel_values`` + ``image_grid_thw`` (images), ``pixel_values_videos`` +
    ``video_grid_thw`` (+ ``second_per_grid_ts``), ``input_features [sum(frames), n_mels]`` + ``feature_lens``
    (audio).  Any may be absent.  A video's temporal positions advance by seconds-per-patch x
    ``position_id_per_seconds``.  Audio tracks interleaved into their video's positions are not built: audio and
    video are separate placeholders."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        super().__init__(cfg, device, dtype)
        ac = cfg.vision.get("audio") or dict(hidden=cfg.vision["hidden"], heads=cfg.vision["heads"],
                                              intermediate=cfg.vision["intermediate"], depth=2)
        self.audio_tower = AudioEncoder(ac, cfg.hidden_size, self.dtype, device)
        self.audio_token_id = cfg.vision.get("audio_token_id", cfg.vocab_size - 2)

    @torch.inference_mode()
    def encode_multimodal_data(self, token_ids, data: dict):
        """Embeddings and prompt rows of every placeholder (image, video, audio) plus M-RoPE positions."""
        embeds, rows, pos, delta = super().encode_multimodal_data(token_ids, data)
        if data.get("input_features") is not None:
            a = self.audio_tower(data["input_features"].to(self.device), list(data["feature_lens"]))
            width = embeds.shape[1]
            if width > a.shape[1]:                      # no deep-stack part
                a = torch.cat([a, a.new_zeros(a.shape[0], width - a.shape[1])], 1)
            aud_rows = [i for i, t in enumerate(token_ids) if t == self.audio_token_id]
            assert len(aud_rows) == a.shape[0], f"{len(aud_rows)} audio placeholders but {a.shape[0]} audio embeddings"
            embeds, rows = torch.cat([embeds, a.to(embeds.dtype)]), rows + aud_rows
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

    _AUDIO = {"conv2d1.weight": "conv1_w", "conv2d1.bias": "conv1_b", "conv2d2.weight": "conv2_w", "conv2d2.bias": "conv2_b",
              "conv2d3.weight": "conv3_w", "conv2d3.bias": "conv3_b"}

    def load_weights(self, weights):
        """Audio tensors: ``audio_tower.layers.N.self_attn.{q,k,v}_proj`` are stacked into the block's ``qkv``;
        ``out_proj`` / ``self_attn_layer_norm`` / ``final_layer_norm`` map to ``proj`` / ``norm1`` / ``norm2``."""
        aud = dict(self.audio_tower.named_parameters())
        rest, loaded = [], set()
        for name, w in weights:
            n = name.removeprefix("thinker.")
            if n.startswith("audio_tower."):
                k = n[len("audio_tower."):]
                k = self._AUDIO.get(k, k).replace("layers.", "blocks.").replace("self_attn_layer_norm.", "norm1.") \
                    .replace("final_layer_norm.", "norm2.").replace("self_attn.out_proj.", "proj.")
                part = None
                for i, key in enumerate(("self_attn.q_proj.", "self_attn.k_proj.", "self_attn.v_proj.")):
                    if key in k:
                        k, part = k.replace(key, "qkv."), i
                if k in aud:
                    if part is None:
                        aud[k].data.copy_(w.reshape(aud[k].shape))
                    else:
                        rows = aud[k].shape[0] // 3
                        aud[k].data[part * rows:(part + 1) * rows].copy_(w)
                    loaded.add(name)
                continue
            rest.append((n.replace("model.language_model.", "model.").replace("model.visual.", "visual."), w))
        return loaded | super().load_weights(rest)
