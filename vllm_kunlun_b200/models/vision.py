"""Vision-language wrappers: a vision tower + projector in front of a registered text decoder.

Reference: ``models/qwen2_vl.py`` / ``qwen2_5_vl.py`` / ``qwen3_vl.py`` (ViT attention through
``flash_attn_varlen_func`` / SDPA ``qwen2_5_vl.py:356-393``, 2-D rotary ``xspeedgate_ops.rope_vit``
``qwen2_vl.py:255``, M-RoPE text positions ``ops/rotary_embedding/kunlun_mrope.py:47-71``) and
``models/internvl.py`` / ``intern_vit.py`` / ``interns1*.py`` (InternViT with SDPA ``intern_vit.py:299``,
pixel-shuffle + MLP projector).

Flow: the engine runs the tower once per request when the request is added, keeps the projected image
embeddings on the device, and during prefill the rows of the step that hold image placeholder tokens are
overwritten with them right after the embedding lookup.  The tower is replicated on every TP rank (it is small
next to the decoder); its GEMMs and attention run on the same kernels as the decoder.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch
import torch.nn as nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from .dense import DenseForCausalLM, GQAAttention
from .layers import RMSNorm, ReplicatedLinear, param


class _Norm(nn.Module):
    def __init__(self, size, eps, kind, dtype, device):
        super().__init__()
        self.kind, self.eps = kind, eps
        self.weight = param(size, dtype=dtype, device=device)
        self.bias = param(size, dtype=dtype, device=device) if kind == "layernorm" else None

    def forward(self, x):
        if self.kind == "layernorm":
            return ops.layernorm(x, self.weight, self.bias, self.eps)
        return ops.rmsnorm(x, self.weight, self.eps)


class VisionBlock(nn.Module):
    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        h, self.heads = vc["hidden"], vc["heads"]
        self.head_dim = h // self.heads
        kind = vc.get("norm", "layernorm")
        self.norm1 = _Norm(h, vc.get("eps", 1e-6), kind, dtype, device)
        self.norm2 = _Norm(h, vc.get("eps", 1e-6), kind, dtype, device)
        self.qkv = ReplicatedLinear(h, 3 * h, bias=True, dtype=dtype, device=device)
        self.proj = ReplicatedLinear(h, h, bias=True, dtype=dtype, device=device)
        self.gated = vc.get("gated_mlp", False)
        inter = vc["intermediate"]
        self.fc1 = ReplicatedLinear(h, inter * (2 if self.gated else 1), bias=True, dtype=dtype, device=device)
        self.fc2 = ReplicatedLinear(inter, h, bias=True, dtype=dtype, device=device)
        self.act = vc.get("act", "quick_gelu")
        self.ls1 = param(h, dtype=dtype, device=device) if vc.get("layer_scale") else None
        self.ls2 = param(h, dtype=dtype, device=device) if vc.get("layer_scale") else None
        # InternViT-6B: RMSNorm of the whole q and k rows (all heads together) before the split
        self.q_norm = RMSNorm(h, vc.get("eps", 1e-6), dtype, device) if vc.get("qk_norm") else None
        self.k_norm = RMSNorm(h, vc.get("eps", 1e-6), dtype, device) if vc.get("qk_norm") else None

    def forward(self, x, cu_seqlens, cos=None, sin=None):
        T = x.shape[0]
        qkv = self.qkv(self.norm1(x)).view(T, 3, self.heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        if self.q_norm is not None:
            q = self.q_norm(q.reshape(T, -1)).view(T, self.heads, self.head_dim)
            k = self.k_norm(k.reshape(T, -1)).view(T, self.heads, self.head_dim)
        if cos is not None:
            q, k = ops.rope_vit(q, k, cos, sin)
        a = ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, self.head_dim ** -0.5)
        a = self.proj(a.reshape(T, -1))
        x = x + (a if self.ls1 is None else a * self.ls1)
        m = self.fc1(self.norm2(x))
        if self.gated:
            m = ops.act_and_mul(m, "silu")
        elif self.act == "quick_gelu":
            m = ops.quick_gelu(m)
        elif self.act == "gelu_tanh":
            m = torch.nn.functional.gelu(m.float(), approximate="tanh").to(m.dtype)
        else:
            m = torch.nn.functional.gelu(m.float()).to(m.dtype)
        m = self.fc2(m)
        return x + (m if self.ls2 is None else m * self.ls2)


class QwenVisionTransformer(nn.Module):
    """Patch embedding (the 3-D conv is a GEMM over flattened patches), 2-D rotary blocks, 2x2 patch merger."""

    def __init__(self, vc: dict, out_hidden: int, dtype, device):
        super().__init__()
        self.vc = vc
        h = vc["hidden"]
        self.patch_dim = vc.get("in_channels", 3) * vc.get("temporal_patch", 2) * vc["patch"] ** 2
        self.patch_embed = ReplicatedLinear(self.patch_dim, h, bias=bool(vc.get("patch_bias")), dtype=dtype, device=device)
        # Qwen3-VL: learned positions on a square table, interpolated bilinearly to every image's grid
        self.num_pos = int(vc.get("num_pos") or 0)
        self.pos_embed = param(self.num_pos, h, dtype=dtype, device=device) if self.num_pos else None
        # Qwen2.5-VL: attention inside windows of window_size pixels, except in the listed blocks
        self.window = int(vc.get("window_size") or 0) // self.merge_of(vc) // vc["patch"] if vc.get("window_size") else 0
        self.fullatt = set(vc.get("fullatt_blocks") or ())
        self.blocks = nn.ModuleList([VisionBlock(vc, dtype, device) for _ in range(vc["depth"])])
        self.merge = vc.get("merge", 2)
        self.ln_q = _Norm(h, vc.get("eps", 1e-6), vc.get("norm", "layernorm"), dtype, device)
        mh = h * self.merge ** 2
        self.merger_fc1 = ReplicatedLinear(mh, mh, bias=True, dtype=dtype, device=device)
        self.merger_fc2 = ReplicatedLinear(mh, out_hidden, bias=True, dtype=dtype, device=device)
        self.head_dim = h // vc["heads"]
        # Qwen3-VL "deep stack": features of intermediate blocks get their own 2x2 mergers and are later added to the
        # decoder's stream after its first layers (models/qwen3_vl.py of the reference, deepstack_visual_indexes)
        self.deepstack_indexes = list(vc.get("deepstack_indexes", ()))
        self.ds_norm = nn.ModuleList([_Norm(mh, vc.get("eps", 1e-6), vc.get("norm", "layernorm"), dtype, device)
                                      for _ in self.deepstack_indexes])
        self.ds_fc1 = nn.ModuleList([ReplicatedLinear(mh, mh, bias=True, dtype=dtype, device=device)
                                     for _ in self.deepstack_indexes])
        self.ds_fc2 = nn.ModuleList([ReplicatedLinear(mh, out_hidden, bias=True, dtype=dtype, device=device)
                                     for _ in self.deepstack_indexes])

    @staticmethod
    def merge_of(vc: dict) -> int:
        return vc.get("merge", 2)

    def window_order(self, grid_thw):
        """Qwen2.5-VL windowed attention: the order of the merged tokens (groups of ``merge^2`` patches) that puts
        every ``window x window`` tile of merged tokens of a frame together, and the cumulative PATCH counts of the
        tiles.  Tiles at the right / bottom edge are partial; like the upstream model, a grid that is an exact
        multiple of the window still gets a (then empty) extra tile row and column, which changes nothing."""
        wz, unit = self.window, self.merge ** 2
        order, cu, base = [], [0], 0
        for t, h, w in grid_thw:
            lh, lw = h // self.merge, w // self.merge
            idx = torch.arange(t * lh * lw).reshape(t, lh, lw)
            ph, pw = wz - lh % wz, wz - lw % wz
            pad = torch.nn.functional.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (lh + ph) // wz, (lw + pw) // wz
            tiles = pad.reshape(t, nh, wz, nw, wz).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, wz * wz)
            counts = (tiles >= 0).sum(1)
            flat = tiles.reshape(-1)
            order.append(flat[flat >= 0] + base)
            for c in counts.tolist():
                if c:
                    cu.append(cu[-1] + c * unit)
            base += t * lh * lw
        return torch.cat(order), torch.tensor(cu, dtype=torch.int32)

    def interpolated_positions(self, grid_thw, device, dtype):
        """Qwen3-VL: the position table (a ``side x side`` square) sampled bilinearly on each image's ``h x w`` grid,
        in the tower's token order (``merge x merge`` windows contiguous), repeated for every frame."""
        side = int(round(self.num_pos ** 0.5))
        table = self.pos_embed.float()
        out = []
        for t, h, w in grid_thw:
            ys = torch.linspace(0, side - 1, h, device=device)
            xs = torch.linspace(0, side - 1, w, device=device)
            y0, x0 = ys.floor().long(), xs.floor().long()
            y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
            fy, fx = (ys - y0).unsqueeze(1), (xs - x0).unsqueeze(0)                    # [h, 1], [1, w]
            def at(yy, xx):
                return table[(yy.unsqueeze(1) * side + xx.unsqueeze(0)).reshape(-1)].reshape(h, w, -1)
            pe = (at(y0, x0) * ((1 - fy) * (1 - fx)).unsqueeze(-1) + at(y0, x1) * ((1 - fy) * fx).unsqueeze(-1)
                  + at(y1, x0) * (fy * (1 - fx)).unsqueeze(-1) + at(y1, x1) * (fy * fx).unsqueeze(-1))
            m = self.merge
            pe = pe.reshape(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(pe.repeat(t, 1))
        return torch.cat(out, 0).to(dtype)

    def rot_pos_emb(self, grid_thw, device):
        """Per-token (h, w) rotary angles; tokens are ordered so that each ``merge x merge`` window is contiguous."""
        m = self.merge
        dim = self.head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        chunks = []
        for t, h, w in grid_thw:
            hp = torch.arange(h).unsqueeze(1).expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            wp = torch.arange(w).unsqueeze(0).expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            ang = torch.cat([hp.unsqueeze(1).float() * inv, wp.unsqueeze(1).float() * inv], -1)  # [h*w, dim]
            chunks.append(ang.repeat(t, 1))
        ang = torch.cat(chunks, 0).to(device)
        return ang.cos(), ang.sin()

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """``pixel_values [n_patches, patch_dim]`` -> ``[n_patches / merge^2, out_hidden * (1 + n_deepstack)]``: the
        main embedding followed by the deep-stack features of the same tokens."""
        grid_thw = [tuple(int(v) for v in g) for g in grid_thw]
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        if self.pos_embed is not None:
            x = x + self.interpolated_positions(grid_thw, x.device, x.dtype)
        cos, sin = self.rot_pos_emb(grid_thw, x.device)
        lens = torch.tensor([h * w for t, h, w in grid_thw for _ in range(t)], dtype=torch.int32)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = lens.cumsum(0)
        cu = cu.to(x.device)
        cu_win, order = None, None
        if self.window:
            # tokens travel through the blocks in window order (whole merge groups move together)
            order, cu_win = self.window_order(grid_thw)
            unit = self.merge ** 2
            order = order.to(x.device)

            def reorder(t):
                return t.reshape(-1, unit, t.shape[-1])[order].reshape(t.shape)
            x, cos, sin = reorder(x), reorder(cos), reorder(sin)
            cu_win = cu_win.to(x.device)
        deep = []
        for li, blk in enumerate(self.blocks):
            x = blk(x, cu if (cu_win is None or li in self.fullatt) else cu_win, cos, sin)
            if li in self.deepstack_indexes:
                k = self.deepstack_indexes.index(li)
                d = self.ds_norm[k](x.reshape(-1, x.shape[-1] * self.merge ** 2))
                d = torch.nn.functional.gelu(self.ds_fc1[k](d).float()).to(x.dtype)
                deep.append(self.ds_fc2[k](d))
        x = self.ln_q(x).reshape(-1, x.shape[-1] * self.merge ** 2)
        x = torch.nn.functional.gelu(self.merger_fc1(x).float()).to(x.dtype)
        x = self.merger_fc2(x)
        if order is not None:
            x = x[torch.argsort(order)]      # back to the image order the prompt's placeholders follow
        return torch.cat([x] + deep, -1) if deep else x


class InternVisionModel(nn.Module):
    """InternViT: class token + learned position embedding, LayerNorm blocks with layer scale, then pixel-shuffle
    down-sampling and the two-layer projector of InternVL."""

    def __init__(self, vc: dict, out_hidden: int, dtype, device):
        super().__init__()
        self.vc = vc
        h = vc["hidden"]
        self.patch_dim = vc.get("in_channels", 3) * vc["patch"] ** 2
        self.patch_embed = ReplicatedLinear(self.patch_dim, h, bias=True, dtype=dtype, device=device)
        self.tokens_per_image = (vc["image_size"] // vc["patch"]) ** 2
        self.cls = param(1, h, dtype=dtype, device=device)
        self.pos = param(self.tokens_per_image + 1, h, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([VisionBlock(vc, dtype, device) for _ in range(vc["depth"])])
        self.ratio = vc.get("downsample", 0.5)
        mh = int(h / self.ratio ** 2)
        self.proj_norm = _Norm(mh, 1e-5, "layernorm", dtype, device)
        self.proj_fc1 = ReplicatedLinear(mh, out_hidden, bias=True, dtype=dtype, device=device)
        self.proj_fc2 = ReplicatedLinear(out_hidden, out_hidden, bias=True, dtype=dtype, device=device)

    def forward(self, pixel_values: torch.Tensor, grid_thw=None) -> torch.Tensor:
        """``pixel_values [n_images, tokens_per_image, patch_dim]`` -> ``[n_images * tokens * ratio^2, out_hidden]``."""
        n, L, _ = pixel_values.shape
        x = self.patch_embed(pixel_values.reshape(n * L, -1).to(self.cls.dtype)).view(n, L, -1)
        x = torch.cat([self.cls.unsqueeze(0).expand(n, 1, -1), x], 1) + self.pos.unsqueeze(0)
        x = x.reshape(n * (L + 1), -1)
        cu = (torch.arange(n + 1, dtype=torch.int32) * (L + 1)).to(x.device)
        for blk in self.blocks:
            x = blk(x, cu)
        x = x.view(n, L + 1, -1)[:, 1:]
        s = int(math.isqrt(L))
        r = int(1 / self.ratio)
        x = x.view(n, s // r, r, s // r, r, -1).permute(0, 1, 3, 2, 4, 5).reshape(n * (s // r) ** 2, -1)  # pixel shuffle
        x = self.proj_fc1(self.proj_norm(x))
        return self.proj_fc2(torch.nn.functional.gelu(x.float()).to(x.dtype))


class MRopeAttention(GQAAttention):
    """Decoder attention with 3-section rotary positions for steps that contain image tokens; text-only steps
    (all decode steps) use the fused 1-D path with positions shifted by the request's M-RoPE delta."""

    def forward(self, hidden):
        ctx = get_forward_context()
        pos3 = ctx.extras.get("mrope_positions")
        if pos3 is None:
            return super().forward(hidden)
        md, cfg = ctx.attn, self.cfg
        qkv = self.qkv_proj(hidden)
        T = qkv.shape[0]
        qs, ks = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        q, k, v = qkv[:, :qs].contiguous(), qkv[:, qs:qs + ks].contiguous(), qkv[:, qs + ks:].contiguous()
        if self.q_norm is not None:
            q = self.q_norm(q.view(-1, self.head_dim)).view(T, qs)
            k = self.k_norm(k.view(-1, self.head_dim)).view(T, ks)
        q, k = ops.mrope(q, k, pos3, self.cos_sin, self.head_dim, list(cfg.mrope_section), cfg.mrope_interleaved)
        kv_cache = ctx.kv_caches[self.layer_idx]
        ops.reshape_and_cache(k.view(T, self.num_kv_heads, self.head_dim), v.view(T, self.num_kv_heads, self.head_dim),
                              kv_cache, md.slot_mapping)
        o = ops.paged_attention(
            q.view(T, self.num_heads, self.head_dim), kv_cache, md.block_tables, md.seq_lens, md.query_start_loc,
            self.scale, md.max_query_len, md.max_seq_len, self.window, self.sinks, md.seq_lens_cpu,
            md.query_start_loc_cpu, workspace=md.workspace, num_decodes=md.num_decodes,
            decode_query_len=1 + md.num_spec_tokens, num_decode_tokens=md.num_decode_tokens)
        return self.o_proj(o.reshape(T, qs))


def get_mrope_positions(token_ids, grid_thw, image_token_id: int, merge: int, video_token_id: Optional[int] = None,
                        video_grid_thw=(), video_t_steps=()):
    """``[3, L]`` (t, h, w) positions and the delta ``next_position - L`` for a prompt whose image placeholders
    (runs of ``image_token_id``) correspond to ``grid_thw`` in order and whose video placeholders (runs of
    ``video_token_id``) to ``video_grid_thw``.  Within a placeholder the height / width axes count merged patches
    and the temporal axis advances by 1 per temporal patch - for a video by ``video_t_steps[i]`` (Qwen2.5-VL:
    seconds per temporal patch x ``tokens_per_second``, truncated after the multiplication); text after it continues
    from the largest position used plus one."""
    L = len(token_ids)
    pos = torch.zeros(3, L, dtype=torch.long)
    grids = {image_token_id: [(g, 1.0) for g in grid_thw or ()]}
    if video_token_id is not None:
        steps = list(video_t_steps) or [1.0] * len(video_grid_thw)
        grids[video_token_id] = list(zip(video_grid_thw, steps))
    used = {k: 0 for k in grids}
    i, nxt = 0, 0
    while i < L:
        tok = token_ids[i]
        if tok in grids and used[tok] < len(grids[tok]):
            (t, h, w), step = grids[tok][used[tok]]
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            tt = (torch.arange(t) * step).long().view(t, 1, 1).expand(t, gh, gw).reshape(-1)
            hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
            ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
            n = min(n, L - i)
            pos[:, i:i + n] = torch.stack([tt, hh, ww])[:, :n] + nxt
            nxt += max(int(tt[-1]) + 1, gh, gw)
            i += n
            used[tok] += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - L


class _VLBase(nn.Module):
    tower_cls = QwenVisionTransformer
    uses_mrope = True

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        super().__init__()
        from . import resolve_model_cls
        self.cfg = cfg
        text_arch = cfg.vision.get("text_architecture", "Qwen2ForCausalLM")
        self.language_model = resolve_model_cls(text_arch)(cfg, device=device, dtype=dtype)
        self.dtype, self.device = self.language_model.dtype, self.language_model.device
        if self.uses_mrope:
            for layer in self.language_model.layers.values():
                # plain attention layers get the three-axis rotary variant; the gated attention of the hybrid decoders
                # handles the positions itself, linear-attention layers have no rotary embedding
                if type(getattr(layer, "self_attn", None)) is GQAAttention:
                    layer.self_attn.__class__ = MRopeAttention
        self.visual = self.tower_cls(cfg.vision, cfg.hidden_size, self.dtype, device)
        self.image_token_id = cfg.vision.get("image_token_id", cfg.vocab_size - 1)
        self.layers = self.language_model.layers
        self.first_layer, self.last_layer = self.language_model.first_layer, self.language_model.last_layer
        self.num_deepstack = len(getattr(self.visual, "deepstack_indexes", ()))
        if self.num_deepstack:
            self.language_model.post_layer_hook = self._deepstack_hook

    def _deepstack_hook(self, layer_idx: int, hidden, residual):
        """After decoder layer ``i < n_deepstack`` the i-th deep-stack feature is added to the stream at the image
        rows of this step (the stream is ``residual + hidden``; ``residual`` is complete on every TP rank)."""
        if layer_idx >= self.num_deepstack or residual is None:
            return
        ex = get_forward_context().extras
        if ex.get("mm_dst") is None:
            return
        H = self.cfg.hidden_size
        feat = ex["mm_src"][:, (1 + layer_idx) * H:(2 + layer_idx) * H].to(residual.dtype)
        residual.index_add_(0, ex["mm_dst"], feat)

    # ---- multimodal
    @torch.inference_mode()
    def embed_multimodal(self, pixel_values, grid_thw=None):
        return self.visual(pixel_values.to(self.device), grid_thw)

    def mm_metadata(self, token_ids, grid_thw):
        """Rows of the prompt to overwrite, and M-RoPE positions when the decoder uses them."""
        rows = [i for i, t in enumerate(token_ids) if t == self.image_token_id]
        if not self.uses_mrope:
            return rows, None, 0
        pos, delta = get_mrope_positions(token_ids, grid_thw, self.image_token_id, self.visual.merge)
        return rows, pos, delta

    def forward(self, input_ids, hidden=None, residual=None):
        lm = self.language_model
        if hidden is None and lm.embed_tokens is not None:
            hidden = lm.embed_tokens(input_ids)
            ex = get_forward_context().extras
            if ex.get("mm_dst") is not None:
                hidden.index_copy_(0, ex["mm_dst"], ex["mm_src"][:, : hidden.shape[1]].to(hidden.dtype))
        return lm(input_ids, hidden, residual)

    def compute_logits(self, hidden):
        return self.language_model.compute_logits(hidden)

    def kv_cache_spec(self, block_size: int):
        return self.language_model.kv_cache_spec(block_size)

    def init_random(self, seed: int = 0, std: float = 0.02):
        self.language_model.init_random(seed, std)
        g = torch.Generator(device=self.device).manual_seed(seed + 77)
        for name, p in self.visual.named_parameters():
            if name.endswith("weight") and p.dim() == 1 and "ls" not in name:
                p.data.fill_(1.0)
            elif name.endswith("bias"):
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g, device=self.device, dtype=torch.float32) * std).to(p.dtype))

    def finish_loading(self):
        self.language_model.finish_loading()

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        text, loaded, original = [], set(), {}
        vis = dict(self.visual.named_parameters())
        for ckpt_name, w in weights:
            name = ckpt_name
            # checkpoints written by transformers 5 nest both halves under ``model.``: ``model.visual.*`` and
            # ``model.language_model.*`` (older ones: ``visual.*`` and ``model.*`` / ``language_model.model.*``)
            if name.startswith("model.visual."):
                name = name[len("model."):]
            elif name.startswith("model.language_model."):
                name = "model." + name[len("model.language_model."):]
            v = self._vision_name(name)
            if v is not None:
                half = None
                if isinstance(v, tuple):        # (parameter, which half of its rows): gate / up of a gated MLP
                    v, half = v
                if v in vis:
                    if half is None:
                        vis[v].data.copy_(w.reshape(vis[v].shape))
                    else:
                        n = vis[v].shape[0] // 2
                        vis[v].data[half * n:(half + 1) * n].copy_(w)
                    loaded.add(ckpt_name)
                continue
            tname = name.replace("language_model.model.", "model.").replace("language_model.", "")
            original[tname] = ckpt_name
            text.append((tname, w))
        # report the checkpoint's own names
        return loaded | {original.get(n, n) for n in self.language_model.load_weights(text)}

    def _vision_name(self, name: str) -> Optional[str]:
        raise NotImplementedError


class QwenVLForConditionalGeneration(_VLBase):
    """Qwen2-VL / Qwen2.5-VL / Qwen3-VL."""

    @torch.inference_mode()
    def encode_multimodal_data(self, token_ids, data: dict):
        """Images (``pixel_values`` + ``image_grid_thw``) and videos (``pixel_values_videos`` + ``video_grid_thw``,
        optionally ``second_per_grid_ts``) of one request: embeddings, the prompt rows they replace, M-RoPE
        positions and the position delta.  Video placeholders are runs of ``video_token_id``; Qwen3-VL prompts carry
        one run per temporal patch (timestamps in between), so each run is a one-frame grid."""
        def grids(key):
            g = data.get(key)
            return [tuple(int(x) for x in r) for r in (g.tolist() if hasattr(g, "tolist") else g)] if g is not None else []

        vc = self.cfg.vision
        ig, vg = grids("image_grid_thw"), grids("video_grid_thw")
        vid_tok = vc.get("video_token_id")
        embeds, rows = [], []
        if data.get("pixel_values") is not None:
            embeds.append(self.visual(data["pixel_values"].to(self.device), ig))
            rows += [i for i, t in enumerate(token_ids) if t == self.image_token_id]
        if data.get("pixel_values_videos") is not None:
            assert vid_tok is not None, "the configuration names no video_token_id"
            embeds.append(self.visual(data["pixel_values_videos"].to(self.device), vg))
            rows += [i for i, t in enumerate(token_ids) if t == vid_tok]
        embeds = torch.cat(embeds) if embeds else torch.zeros(0, self.cfg.hidden_size * (1 + self.num_deepstack),
                                                               dtype=self.dtype, device=self.device)
        assert len(rows) == embeds.shape[0], f"{len(rows)} placeholder tokens but {embeds.shape[0]} embeddings"
        steps = []
        if vc.get("video_frame_runs"):
            vg = [(1, h, w) for t, h, w in vg for _ in range(t)]
        elif vc.get("tokens_per_second"):
            sec = data.get("second_per_grid_ts")
            sec = [float(x) for x in sec] if sec is not None else [1.0] * len(vg)
            steps = [x * vc["tokens_per_second"] for x in sec]
        pos, delta = get_mrope_positions(token_ids, ig, self.image_token_id, self.visual.merge, vid_tok, vg, steps)
        return embeds, rows, pos, delta

    _MAP = {"patch_embed.proj.weight": "patch_embed.weight", "patch_embed.proj.bias": "patch_embed.bias",
            "pos_embed.weight": "pos_embed", "attn.qkv.": "qkv.", "attn.proj.": "proj.",
            "mlp.fc1.": "fc1.", "mlp.fc2.": "fc2.", "mlp.linear_fc1.": "fc1.", "mlp.linear_fc2.": "fc2.",
            "mlp.down_proj.": "fc2.", "merger.ln_q.": "ln_q.", "merger.mlp.0.": "merger_fc1.",
            "merger.mlp.2.": "merger_fc2.", "deepstack_merger_list.": "ds_", "merger.norm.": "ln_q.",
            "merger.linear_fc1.": "merger_fc1.", "merger.linear_fc2.": "merger_fc2."}

    def _vision_name(self, name):
        if not name.startswith("visual."):
            return None
        n = name[len("visual."):]
        for half, key in enumerate(("mlp.gate_proj.", "mlp.up_proj.")):     # Qwen2.5-VL: gate | up stacked in fc1
            if key in n:
                return n.replace(key, "fc1."), half
        for a, b in self._MAP.items():
            n = n.replace(a, b)
        import re
        # deepstack_merger_list.<k>.{norm,linear_fc1,linear_fc2}.* -> ds_{norm,fc1,fc2}.<k>.*
        # (Qwen3-Omni: merger_list.<k>.{ln_q,mlp.0,mlp.2}.*)
        m = re.match(r"(?:ds_|merger_list\.)(\d+)\.(norm|linear_fc1|linear_fc2|ln_q|mlp\.0|mlp\.2)\.(.*)", n)
        if m:
            kind = {"norm": "ds_norm", "linear_fc1": "ds_fc1", "linear_fc2": "ds_fc2", "ln_q": "ds_norm",
                    "mlp.0": "ds_fc1", "mlp.2": "ds_fc2"}[m.group(2)]
            return f"{kind}.{m.group(1)}.{m.group(3)}"
        return n


class Qwen3_5ForConditionalGeneration(QwenVLForConditionalGeneration):
    """Qwen3.5 / Qwen3.5-MoE with images and videos (``models/qwen3_5.py:627-700`` of the reference): the Qwen3-VL tower
    (no deep-stack features) in front of the hybrid gated-delta-net decoder; interleaved M-RoPE over the rotated
    quarter of each head in the full-attention layers."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        cfg.vision.setdefault("text_architecture", "Qwen3_5MoeForCausalLM" if cfg.num_experts else "Qwen3_5ForCausalLM")
        super().__init__(cfg, device, dtype)

    def state_cache_spec(self):
        return self.language_model.state_cache_spec()

    @property
    def uses_state_cache(self) -> bool:
        return self.language_model.uses_state_cache


class Qwen3VLMoeForConditionalGeneration(QwenVLForConditionalGeneration):
    """Qwen3-VL with the Qwen3-MoE decoder (``models/qwen3_vl_moe.py`` of the reference): the same tower with
    deep-stack features, the text side is the sparse-MoE decoder of this package."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        cfg.vision.setdefault("text_architecture", "Qwen3MoeForCausalLM")
        if cfg.vision["text_architecture"] in ("Qwen3ForCausalLM", "Qwen2ForCausalLM") and cfg.num_experts:
            cfg.vision["text_architecture"] = "Qwen3MoeForCausalLM"
        super().__init__(cfg, device, dtype)


class InternVLChatModel(_VLBase):
    """InternVL / Intern-S1: InternViT tower, pixel-shuffle projector, 1-D rotary decoder."""

    tower_cls = InternVisionModel
    uses_mrope = False

    _MAP = {"vision_model.embeddings.patch_embedding.": "patch_embed.", "vision_model.embeddings.class_embedding": "cls",
            "vision_model.embeddings.position_embedding": "pos", "vision_model.encoder.layers.": "blocks.",
            ".attn.qkv.": ".qkv.", ".attn.proj.": ".proj.", ".mlp.fc1.": ".fc1.", ".mlp.fc2.": ".fc2.",
            "mlp1.0.": "proj_norm.", "mlp1.1.": "proj_fc1.", "mlp1.3.": "proj_fc2.",
            # checkpoints in the transformers-native layout (InternVLForConditionalGeneration)
            "vision_tower.embeddings.cls_token": "cls", "vision_tower.embeddings.position_embeddings": "pos",
            "vision_tower.embeddings.patch_embeddings.projection.": "patch_embed.",
            "vision_tower.encoder.layer.": "blocks.", ".attention.qkv.": ".qkv.",
            ".attention.projection_layer.": ".proj.", ".attention.q_norm.": ".q_norm.", ".attention.k_norm.": ".k_norm.",
            ".layernorm_before.": ".norm1.", ".layernorm_after.": ".norm2.", ".lambda_1": ".ls1", ".lambda_2": ".ls2",
            "multi_modal_projector.layer_norm.": "proj_norm.", "multi_modal_projector.linear_1.": "proj_fc1.",
            "multi_modal_projector.linear_2.": "proj_fc2."}

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        super().__init__(cfg, device, dtype)
        for n, p_ in self.visual.named_parameters():     # checkpoints without attention biases leave these at zero
            if n.endswith(".bias"):
                p_.data.zero_()

    def _vision_name(self, name):
        if not name.startswith(("vision_model.", "mlp1.", "vision_tower.", "multi_modal_projector.")):
            return None
        n = name
        for a, b in self._MAP.items():
            n = n.replace(a, b)
        return n

    def load_weights(self, weights):
        """The transformers-native layout keeps q / k / v of the tower apart: they are stacked into ``qkv`` here;
        ``model.vision_tower.*`` / ``model.multi_modal_projector.*`` / ``model.language_model.*`` lose the prefix."""
        out, parts, original = [], {}, {}
        for name, w in weights:
            n = name
            if n.startswith("model.") and not n.startswith("model.layers.") and not n.startswith("model.embed_tokens.") \
                    and not n.startswith("model.norm."):
                n = n[len("model."):]
                if n.startswith("language_model."):
                    n = "model." + n[len("language_model."):]
            hit = next((x for x in (".attention.q_proj.", ".attention.k_proj.", ".attention.v_proj.") if x in n), None)
            if hit is not None and n.startswith("vision_tower."):
                key = n.replace(hit, ".attention.qkv.")
                got = parts.setdefault(key, {})
                got[hit] = (name, w)
                if len(got) == 3:
                    out.append((key, torch.cat([got[x][1] for x in (".attention.q_proj.", ".attention.k_proj.", ".attention.v_proj.")])))
                    original[key] = [got[x][0] for x in got]
                continue
            original[n] = [name]
            out.append((n, w))
        loaded = super().load_weights(out)
        return {o for g in loaded for o in original.get(g, [g])}


class _ClippedLinear(nn.Module):
    """Bias-free linear whose input and output are clamped to learned ranges (checkpoint buffers ``input_min`` /
    ``input_max`` / ``output_min`` / ``output_max``; infinite when the checkpoint has none)."""

    def __init__(self, n_in: int, n_out: int, dtype, device):
        super().__init__()
        self.linear = ReplicatedLinear(n_in, n_out, bias=False, dtype=dtype, device=device)
        self.clip = [-math.inf, math.inf, -math.inf, math.inf]      # host floats: no device read in forward
        self.clipped = False

    def forward(self, x):
        if not self.clipped:
            return self.linear(x)
        c = self.clip
        return self.linear(x.clamp(c[0], c[1])).clamp(c[2], c[3])


class Gemma4VisionBlock(nn.Module):
    """Encoder layer of the Gemma-4 tower: sandwich RMSNorms (weights multiply directly), q / k RMSNorm per head, V
    RMS-normalised without a weight, softmax scale 1, rotary embedding over the patch's (x, y) position - the first
    half of a head rotates with x, the second with y - and a gated tanh-GELU MLP."""

    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        h, self.heads, self.kv_heads = vc["hidden"], vc["heads"], vc.get("kv_heads") or vc["heads"]
        self.head_dim = vc.get("head_dim") or h // self.heads
        eps = self.eps = vc.get("eps", 1e-6)
        lin = lambda a, b: _ClippedLinear(a, b, dtype, device)  # noqa: E731
        self.q_proj, self.k_proj = lin(h, self.heads * self.head_dim), lin(h, self.kv_heads * self.head_dim)
        self.v_proj, self.o_proj = lin(h, self.kv_heads * self.head_dim), lin(self.heads * self.head_dim, h)
        self.q_norm = RMSNorm(self.head_dim, eps, dtype, device)
        self.k_norm = RMSNorm(self.head_dim, eps, dtype, device)
        self.gate_proj, self.up_proj = lin(h, vc["intermediate"]), lin(h, vc["intermediate"])
        self.down_proj = lin(vc["intermediate"], h)
        self.input_layernorm, self.post_attention_layernorm = RMSNorm(h, eps, dtype, device), RMSNorm(h, eps, dtype, device)
        self.pre_feedforward_layernorm = RMSNorm(h, eps, dtype, device)
        self.post_feedforward_layernorm = RMSNorm(h, eps, dtype, device)

    @staticmethod
    def _rope2d(x, cos, sin):
        """``x [T, heads, D]``; ``cos`` / ``sin [T, D]``: two halves of ``D / 2`` channels, each rotated split-half."""
        D = x.shape[-1]
        part = 2 * (D // 4)
        out = []
        for k in range(2):
            xp = x[..., k * part:(k + 1) * part].float()
            c, s_ = cos[:, None, k * part:(k + 1) * part], sin[:, None, k * part:(k + 1) * part]
            x1, x2 = xp[..., :part // 2], xp[..., part // 2:]
            out.append(xp * c + torch.cat([-x2, x1], -1) * s_)
        if 2 * part < D:
            out.append(x[..., 2 * part:].float())
        return torch.cat(out, -1).to(x.dtype)

    def forward(self, x, cu_seqlens, cos, sin):
        T = x.shape[0]
        h = self.input_layernorm(x)
        q = self.q_norm(self.q_proj(h).view(T * self.heads, self.head_dim)).view(T, self.heads, self.head_dim)
        k = self.k_norm(self.k_proj(h).view(T * self.kv_heads, self.head_dim)).view(T, self.kv_heads, self.head_dim)
        v = self.v_proj(h).view(T, self.kv_heads, self.head_dim).float()
        v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        q, k = self._rope2d(q, cos, sin), self._rope2d(k, cos, sin)
        if self.kv_heads != self.heads:
            rep = self.heads // self.kv_heads
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        a = ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, 1.0)
        x = x + self.post_attention_layernorm(self.o_proj(a.reshape(T, -1)))
        h = self.pre_feedforward_layernorm(x)
        m = torch.nn.functional.gelu(self.gate_proj(h).float(), approximate="tanh").to(h.dtype) * self.up_proj(h)
        return x + self.post_feedforward_layernorm(self.down_proj(m))


class GemmaVisionTower(nn.Module):
    """Gemma-4 vision tower (``models/gemma4_mm.py`` of the reference drives upstream's tower of the same design):
    patches (values in [0, 1], rescaled to [-1, 1]) are projected without a bias and get the sum of two learned
    position rows - one looked up by the patch's x, one by its y; encoder layers with 2-D rotary embedding;
    ``pool x pool`` patches are averaged into one soft token, scaled by ``sqrt(hidden)``, optionally standardised
    with learned statistics; then an RMS norm without a weight and the projection into the decoder width."""

    def __init__(self, vc: dict, out_hidden: int, dtype, device):
        super().__init__()
        self.vc = vc
        h = vc["hidden"]
        self.patch_dim = vc.get("in_channels", 3) * vc["patch"] ** 2
        self.input_proj = ReplicatedLinear(self.patch_dim, h, bias=False, dtype=dtype, device=device)
        self.position_embedding_table = param(2, vc.get("position_embedding_size", 10240), h, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([Gemma4VisionBlock(vc, dtype, device) for _ in range(vc["depth"])])
        self.pool = vc.get("pool", 3)
        self.standardize = bool(vc.get("standardize"))
        if self.standardize:
            self.std_bias, self.std_scale = param(h, dtype=dtype, device=device), param(h, dtype=dtype, device=device)
        self.proj = ReplicatedLinear(h, out_hidden, bias=False, dtype=dtype, device=device)
        self.eps = vc.get("eps", 1e-6)
        self.theta = float(vc.get("rope_theta", 100.0))
        self.head_dim = vc.get("head_dim") or h // vc["heads"]
        self.merge = 1

    def tokens_per_image(self, grid) -> int:
        _, gh, gw = grid
        return (gh // self.pool) * (gw // self.pool)

    def forward(self, pixel_values: torch.Tensor, grid_thw=None) -> torch.Tensor:
        """``pixel_values [sum(h * w), patch_dim]`` (patches of every image row-major, values in [0, 1]) and the
        patch grids ``[(1, h, w), ...]`` (``h``, ``w`` multiples of the pooling size) -> ``[sum(h * w / pool^2),
        out_hidden]``."""
        if pixel_values.dim() == 3:      # [n_images, patches, patch_dim] of equal square images
            n, L, _ = pixel_values.shape
            side = int(math.isqrt(L))
            grid_thw = grid_thw or [(1, side, side)] * n
            pixel_values = pixel_values.reshape(n * L, -1)
        dt, dev = self.input_proj.weight.dtype, pixel_values.device
        xs, ys = [], []
        for _, gh, gw in grid_thw:
            ys.append(torch.arange(gh, device=dev).repeat_interleave(gw))
            xs.append(torch.arange(gw, device=dev).repeat(gh))
        px, py = torch.cat(xs), torch.cat(ys)
        x = self.input_proj((2.0 * (pixel_values.float() - 0.5)).to(dt))
        x = x + self.position_embedding_table[0, px] + self.position_embedding_table[1, py]
        half = self.head_dim // 2        # channels per axis; frequencies as for a head of that size
        inv = 1.0 / (self.theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=dev) / half))
        fx, fy = px[:, None].float() * inv[None], py[:, None].float() * inv[None]
        ang = torch.cat([fx, fx, fy, fy], -1)
        cos, sin = ang.cos(), ang.sin()
        lens = [gh * gw for _, gh, gw in grid_thw]
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        cu = cu.to(dev)
        for blk in self.blocks:
            x = blk(x, cu, cos, sin)
        k, outs, o = self.pool, [], 0
        for (_, gh, gw), n in zip(grid_thw, lens):
            img = x[o:o + n].view(gh // k, k, gw // k, k, -1).float().mean((1, 3))
            outs.append(img.reshape((gh // k) * (gw // k), -1))
            o += n
        x = torch.cat(outs) * (x.shape[-1] ** 0.5)
        if self.standardize:
            x = (x - self.std_bias.float()) * self.std_scale.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.proj(x.to(dt))


class Gemma4ForConditionalGeneration(_VLBase):
    """Gemma-4 with the vision tower (``Gemma4ForConditionalGeneration``, ``models/gemma4_mm.py`` in the reference):
    image soft tokens replace the placeholder embeddings AFTER the embedding scale, 1-D rotary positions, and the
    per-layer token embedding of a placeholder row is the padding token's.  Image rows attend causally, as in
    the reference (the training-time mask lets the soft tokens of one image see each other in the sliding layers).
    The audio tower of the any-to-any checkpoints is not built: their audio tensors are skipped."""

    tower_cls = GemmaVisionTower
    uses_mrope = False

    _MAP = {"vision_tower.patch_embedder.input_proj.": "input_proj.",
            "vision_tower.patch_embedder.position_embedding_table": "position_embedding_table",
            "vision_tower.encoder.layers.": "blocks.", ".self_attn.": ".", ".mlp.": ".",
            "vision_tower.std_bias": "std_bias", "vision_tower.std_scale": "std_scale",
            "embed_vision.embedding_projection.": "proj."}

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        cfg.vision.setdefault("text_architecture", "Gemma4ForCausalLM")
        super().__init__(cfg, device, dtype)
        self.language_model.input_embeds_hook = self._inject

    def _inject(self, hidden):
        """-> (embeddings with the soft tokens in place, the rows they went to or None)."""
        ex = get_forward_context().extras
        if ex.get("mm_dst") is None:
            return hidden, None
        hidden = hidden.clone()
        hidden.index_copy_(0, ex["mm_dst"], ex["mm_src"][:, : hidden.shape[1]].to(hidden.dtype))
        return hidden, ex["mm_dst"]

    def forward(self, input_ids, hidden=None, residual=None):
        return self.language_model(input_ids, hidden, residual)  # injection happens inside, after the embed scale

    def _vision_name(self, name):
        if not (name.startswith("vision_tower.") or name.startswith("embed_vision.")):
            return None
        n = name
        for a, b in self._MAP.items():
            n = n.replace(a, b)
        return n

    def load_weights(self, weights):
        """Besides the tensors: the clipping ranges of the tower's linears (scalars ``*.input_min`` ...), kept in each
        linear's ``clip`` buffer; audio tensors are skipped.  Returns the checkpoint names that were used."""
        slot = {"input_min": 0, "input_max": 1, "output_min": 2, "output_max": 3}
        mods = dict(self.visual.named_modules())
        keep, original, loaded = [], {}, set()
        for name, w in weights:
            n = name.removeprefix("model.")
            if n.startswith("audio_tower.") or n.startswith("embed_audio."):
                continue
            stem, _, leaf = n.rpartition(".")
            if n.startswith("vision_tower.") and leaf in slot:
                m = mods.get(self._vision_name(stem))
                if m is not None:
                    m.clip[slot[leaf]] = float(w)
                    m.clipped = any(math.isfinite(v) for v in m.clip)
                    loaded.add(name)
                continue
            if n.startswith("language_model."):
                n = "model." + n[len("language_model."):]
            elif not (n.startswith("vision_tower.") or n.startswith("embed_vision.")):
                n = name
            original[n] = name
            keep.append((n, w))
        return loaded | {original.get(g, g) for g in super().load_weights(keep)}
