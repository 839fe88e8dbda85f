"""fp32 PyTorch oracles: normalisation, activation, rotary, quantisation.

Each function restates the math of one device op of the reference plugin (whose
kernels live in closed libraries); the reference binding site is cited per
function.  These run on CPU and are the ground truth for every CUDA kernel test.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

FP8_MAX = 448.0  # e4m3fn


# ----------------------------------------------------------------------------- norms

def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool = False) -> torch.Tensor:
    """``_C::rmsnorm`` / ``_C::gemma_rmsnorm`` (``ops/_custom_ops.py:303-340,525-555``)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    w = weight.float() + 1.0 if gemma else weight.float()
    return (xf * torch.rsqrt(var + eps) * w).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                gemma: bool = False):
    """``_C::add_rmsnorm`` (``ops/_custom_ops.py:255-300``): ``res = x + res; out = norm(res)``.

    Returns ``(out, new_residual)``; the sum is rounded to the activation dtype
    before normalising, as the in-place device op does."""
    s = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(s, weight, eps, gemma), s


def rms_norm_gated(x, z, weight, eps: float, norm_before_gate: bool = True, group_size: Optional[int] = None):
    """``_C::rms_norm_gated`` (``ops/fla/layernorm_guard.py:54-56``)."""
    xf, zf = x.float(), z.float()
    if not norm_before_gate:
        xf = xf * torch.nn.functional.silu(zf)
    shp = xf.shape
    if group_size is not None:
        xf = xf.reshape(*shp[:-1], shp[-1] // group_size, group_size)
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    xf = xf.reshape(shp) * weight.float()
    if norm_before_gate:
        xf = xf * torch.nn.functional.silu(zf)
    return xf.to(x.dtype)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``kunlun_ops.l2norm`` (``ops/fla/l2norm.py:21``)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def layernorm(x, weight, bias, eps):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight.float(),
                                          None if bias is None else bias.float(), eps).to(x.dtype)


# ----------------------------------------------------------------------------- activations

def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """``_C::silu_and_mul`` (``ops/_custom_ops.py:699-716``)."""
    d = x.shape[-1] // 2
    xf = x.float()
    return (torch.nn.functional.silu(xf[..., :d]) * xf[..., d:]).to(x.dtype)


def swigluoai_and_mul(x: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """``_C::swigluoai_and_mul`` (``ops/_custom_ops.py:728-759``): interleaved gate/up, clamped."""
    xf = x.float()
    gate, up = xf[..., ::2], xf[..., 1::2]
    gate = gate.clamp(max=limit)
    up = up.clamp(min=-limit, max=limit)
    return ((up + 1.0) * gate * torch.sigmoid(alpha * gate)).to(x.dtype)


def quick_gelu(x: torch.Tensor) -> torch.Tensor:
    """``KunlunOps.quick_gelu`` (``ops/_kunlun_ops.py:145-151``)."""
    xf = x.float()
    return (xf * torch.sigmoid(1.702 * xf)).to(x.dtype)


def gelu_tanh_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    xf = x.float()
    return (torch.nn.functional.gelu(xf[..., :d], approximate="tanh") * xf[..., d:]).to(x.dtype)


def fused_gdn_gating(A_log, a, dt_bias, beta: float = 1.0, threshold: float = 20.0):
    """``kunlun_ops.fused_gdn_gating`` (``ops/_kunlun_ops.py:772-785``): ``g = -exp(A_log) * softplus(a + dt_bias)``."""
    return -torch.exp(A_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float(), beta, threshold)


def apply_repetition_penalties(logits, prompt_mask, output_mask, penalties):
    """``_C::apply_repetition_penalties_`` (``ops/_custom_ops.py:1957-1971``)."""
    seen = prompt_mask | output_mask
    p = penalties.float().unsqueeze(1).expand_as(logits)
    lf = logits.float()
    scaled = torch.where(lf > 0, lf / p, lf * p)
    return torch.where(seen, scaled, lf).to(logits.dtype)


# ----------------------------------------------------------------------------- rotary

def _yarn_find_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1.0:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


def rope_inv_freq(rotary_dim: int, theta: float, scaling=None) -> tuple[torch.Tensor, float]:
    """Inverse frequencies and the cos/sin magnitude scale for plain / linear / llama3 / YaRN RoPE.

    YaRN follows ``DeepseekScalingRotaryEmbedding`` as used at
    ``models/deepseek_v2.py:889-903`` of the reference."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    mscale = 1.0
    if scaling is None or scaling.type == "none":
        return inv, mscale
    if scaling.type == "linear":
        return inv / scaling.factor, mscale
    if scaling.type == "llama3":
        low = scaling.original_max_position / scaling.low_freq_factor
        high = scaling.original_max_position / scaling.high_freq_factor
        wavelen = 2 * math.pi / inv
        smooth = (scaling.original_max_position / wavelen - scaling.low_freq_factor) / (
            scaling.high_freq_factor - scaling.low_freq_factor)
        out = torch.where(wavelen > low, inv / scaling.factor, inv)
        mid = (wavelen <= low) & (wavelen >= high)
        out = torch.where(mid, (1 - smooth) * inv / scaling.factor + smooth * inv, out)
        return out, mscale
    if scaling.type == "proportional":
        # the first ``partial`` of the head's angle pairs rotate with exponents relative to the whole head; the other
        # pairs keep angle 0 (cos 1, sin 0: they pass through)
        n_rot = int(scaling.partial * rotary_dim // 2)
        out = torch.zeros(rotary_dim // 2, dtype=torch.float32)
        out[:n_rot] = 1.0 / (theta ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32) / rotary_dim))
        return out / scaling.factor, mscale
    if scaling.type == "yarn":
        lo = _yarn_find_dim(scaling.beta_fast, rotary_dim, theta, scaling.original_max_position)
        hi = _yarn_find_dim(scaling.beta_slow, rotary_dim, theta, scaling.original_max_position)
        if getattr(scaling, "truncate", True):      # whole dimensions (DeepSeek); gpt-oss keeps the fractions
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rotary_dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
        mask = 1.0 - ramp
        out = inv / scaling.factor * (1 - mask) + inv * mask

        def _ms(scale, m):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
        mscale = _ms(scaling.factor, scaling.mscale) / _ms(scaling.factor, scaling.mscale_all_dim)
        return out, mscale
    raise ValueError(f"unknown rope scaling {scaling.type}")


def build_cos_sin_cache(rotary_dim: int, max_pos: int, theta: float, scaling=None) -> torch.Tensor:
    """``[max_pos, rotary_dim]`` fp32 cache: first half cos, second half sin (the layout
    ``_C::rotary_embedding`` reads, ``ops/_custom_ops.py:993-1028``)."""
    inv, mscale = rope_inv_freq(rotary_dim, theta, scaling)
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
               head_dim: int, neox: bool = True, rotary_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate ``x [T, H*head_dim]`` (or ``[T, H, head_dim]``) at ``positions [T]``."""
    shp = x.shape
    T = positions.shape[0]
    xf = x.float().reshape(T, -1, head_dim)
    rd = rotary_dim or cos_sin_cache.shape[-1]
    cs = cos_sin_cache[positions.long()].float()
    cos, sin = cs[:, : rd // 2].unsqueeze(1), cs[:, rd // 2: rd].unsqueeze(1)
    rot, rest = xf[..., :rd], xf[..., rd:]
    if neox:
        x1, x2 = rot[..., : rd // 2], rot[..., rd // 2:]
        o = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    else:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
        o = torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
    return torch.cat([o, rest], dim=-1).reshape(shp).to(x.dtype)


def apply_mrope(x, positions3, cos_sin_cache, head_dim, sections, interleaved: bool = False):
    """3-section multimodal RoPE (``ops/rotary_embedding/kunlun_mrope.py:47-71``).

    ``positions3 [3, T]`` holds temporal/height/width positions; ``sections`` partitions the
    ``rotary_dim/2`` frequency slots among them."""
    T = positions3.shape[1]
    rd = cos_sin_cache.shape[-1]
    half = rd // 2
    cs = cos_sin_cache[positions3.long()].float()  # [3, T, rd]
    cos3, sin3 = cs[..., :half], cs[..., half:]
    if interleaved:
        sel = torch.zeros(half, dtype=torch.long)
        for axis in (1, 2):
            idx = torch.arange(axis, sections[axis] * 3, 3)
            sel[idx[idx < half]] = axis      # slots past the rotary width do not exist (small heads)
    else:
        sel = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sections)])
    ar = torch.arange(half)
    cos = cos3[sel, :, ar].transpose(0, 1).unsqueeze(1)  # [T,1,half]
    sin = sin3[sel, :, ar].transpose(0, 1).unsqueeze(1)
    shp = x.shape
    xf = x.float().reshape(T, -1, head_dim)
    rot, rest = xf[..., :rd], xf[..., rd:]
    x1, x2 = rot[..., :half], rot[..., half:]
    o = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    return torch.cat([o, rest], dim=-1).reshape(shp).to(x.dtype)


def split_qknorm_rope(qkv, positions, cos_sin_cache, q_weight, k_weight, eps,
                      num_heads, num_kv_heads, head_dim, neox=True, gemma=False):
    """``_C::split_norm_rope_neox`` (``ops/_custom_ops.py:577-646``): split a fused qkv row,
    per-head RMSNorm on q and k, then RoPE.  Returns ``(q, k, v)``."""
    T = qkv.shape[0]
    qs, ks = num_heads * head_dim, num_kv_heads * head_dim
    q, k, v = qkv[:, :qs], qkv[:, qs:qs + ks], qkv[:, qs + ks:]
    if q_weight is not None:
        q = rmsnorm(q.reshape(T, num_heads, head_dim), q_weight, eps, gemma).reshape(T, qs)
        k = rmsnorm(k.reshape(T, num_kv_heads, head_dim), k_weight, eps, gemma).reshape(T, ks)
    q = apply_rope(q, positions, cos_sin_cache, head_dim, neox)
    k = apply_rope(k, positions, cos_sin_cache, head_dim, neox)
    return q, k, v.contiguous()


# ----------------------------------------------------------------------------- quantisation

def quant_fp8_per_group(x: torch.Tensor, group: int = 128, ue8m0: bool = False):
    """Dynamic per-token-group (1 x ``group``) e4m3 quantisation.  Returns ``(q_fp8, scale_fp32)``
    with ``x ~= q * scale``; scales are ``[..., K/group]``.  This is the activation format of
    the fp8 block-scaled GEMM."""
    shp = x.shape
    xf = x.float().reshape(*shp[:-1], shp[-1] // group, group)
    amax = xf.abs().amax(-1, keepdim=True).clamp(min=1e-10)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shp), scale.squeeze(-1)


def quant_fp8_block(w: torch.Tensor, block=(128, 128)):
    """Per-block (128 x 128) absmax e4m3 weight quantisation.  Returns ``(w_fp8, scale_inv)``
    with ``w ~= w_fp8 * scale_inv[block]`` - the ``weight_scale_inv`` checkpoint convention
    (``ops/linear.py:91-96`` shards these scales)."""
    N, K = w.shape[-2:]
    bn, bk = block
    Np, Kp = -(-N // bn) * bn, -(-K // bk) * bk
    wf = torch.zeros(*w.shape[:-2], Np, Kp, dtype=torch.float32)
    wf[..., :N, :K] = w.float()
    v = wf.reshape(*w.shape[:-2], Np // bn, bn, Kp // bk, bk)
    amax = v.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-10)
    scale = amax / FP8_MAX
    q = (v / scale).clamp(-FP8_MAX, FP8_MAX).reshape(*w.shape[:-2], Np, Kp)[..., :N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.squeeze(-1).squeeze(-2).contiguous()


def dequant_fp8_block(w_fp8: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    N, K = w_fp8.shape[-2:]
    bn, bk = block
    s = scale_inv.float().repeat_interleave(bn, -2).repeat_interleave(bk, -1)[..., :N, :K]
    return w_fp8.float() * s


def fp8_block_gemm(x_q, x_scale, w_fp8, w_scale_inv, block=(128, 128), out_dtype=torch.bfloat16):
    """``out = (x_q * x_scale) @ (w_fp8 * w_scale_inv).T`` with per-K-block promotion in fp32."""
    K = x_q.shape[-1]
    xs = x_scale.float().repeat_interleave(block[1], -1)[..., :K]
    xf = x_q.float() * xs
    return (xf @ dequant_fp8_block(w_fp8, w_scale_inv, block).T).to(out_dtype)


def quant_fp8_static(x, scale):
    return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def quant_int8_per_token(x: torch.Tensor):
    """``_C::scaled_int8_quant`` dynamic path (``ops/_custom_ops.py:1633-1685``)."""
    xf = x.float()
    amax = xf.abs().amax(-1, keepdim=True).clamp(min=1e-10)
    scale = amax / 127.0
    q = torch.round(xf / scale).clamp(-128, 127).to(torch.int8)
    return q, scale


def quant_int8_static(x, scale):
    return torch.round(x.float() / scale).clamp(-128, 127).to(torch.int8)


def int8_scaled_mm(a_q, a_scale, w_q, w_scale, bias=None, out_dtype=torch.bfloat16, azp_adj=None, azp=None):
    """``_C::cutlass_scaled_mm(_azp)`` / ``_C::matmul`` (``ops/_custom_ops.py:1707-1883``):
    ``out = a_scale * (a_q @ w_q.T) * w_scale (+ bias)`` with int32 accumulation."""
    acc = a_q.to(torch.int32).float() @ w_q.to(torch.int32).float().T
    if azp_adj is not None:
        acc = acc - (azp_adj.float() if azp is None else azp.float() * azp_adj.float())
    out = acc * a_scale.float() * w_scale.float().reshape(1, -1)
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)


# AWQ packs eight 4-bit values per int32 in the order [0, 2, 4, 6, 1, 3, 5, 7].
AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)


def awq_dequantize(qweight, scales, qzeros, group_size: int):
    """``_C::awq_dequantize`` (``ops/_custom_ops.py:1416-1440``).  ``qweight [K, N/8]`` int32,
    ``qzeros [K/g, N/8]`` int32, ``scales [K/g, N]``.  Returns ``[K, N]``."""
    shifts = torch.tensor([4 * i for i in AWQ_ORDER], dtype=torch.int32)
    w = ((qweight.unsqueeze(-1) >> shifts) & 0xF).reshape(qweight.shape[0], -1)
    z = ((qzeros.unsqueeze(-1) >> shifts) & 0xF).reshape(qzeros.shape[0], -1)
    z = z.repeat_interleave(group_size, 0)[: w.shape[0]]
    s = scales.float().repeat_interleave(group_size, 0)[: w.shape[0]]
    return ((w - z).float() * s).to(scales.dtype)


def awq_pack(w_int: torch.Tensor) -> torch.Tensor:
    """Inverse of the unpacking above: ``[K, N]`` values in ``0..15`` -> ``[K, N/8]`` int32."""
    K, N = w_int.shape
    v = w_int.reshape(K, N // 8, 8).to(torch.int64)
    out = torch.zeros(K, N // 8, dtype=torch.int64)
    for pos, src in enumerate(AWQ_ORDER):
        out |= (v[..., pos] & 0xF) << (4 * src)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def gptq_dequantize(qweight, scales, qzeros, g_idx, bits: int = 4):
    """GPTQ (``quantization/gptq.py:68-143``): ``qweight [K/pack, N]`` packed along K,
    ``qzeros [K/g, N/pack]`` packed along N with the +1 zero-point convention."""
    pack = 32 // bits
    mask = (1 << bits) - 1
    shifts = torch.arange(0, 32, bits, dtype=torch.int32)
    w = ((qweight.unsqueeze(1) >> shifts.view(1, -1, 1)) & mask).reshape(-1, qweight.shape[1])
    z = ((qzeros.unsqueeze(-1) >> shifts) & mask).reshape(qzeros.shape[0], -1) + 1
    K = w.shape[0]
    if g_idx is None:
        g = scales.shape[0]
        g_idx = torch.arange(K) // (K // g)
    return ((w - z[g_idx.long()]).float() * scales.float()[g_idx.long()]).to(scales.dtype)


def linear(x, weight, bias=None):
    out = x.float() @ weight.float().T
    if bias is not None:
        out = out + bias.float()
    return out.to(x.dtype)
