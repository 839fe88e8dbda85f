"""fp32 PyTorch oracles: sampling, rejection sampling, gated delta-net, causal conv, LoRA."""
from __future__ import annotations

from typing import Optional

import torch

PLACEHOLDER_TOKEN_ID = -1


# ----------------------------------------------------------------------------- sampling

def apply_top_k_top_p(logits, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor]):
    """Sort-based masking, the native fallback of ``TopKTopPSampler``
    (``v1/sample/ops/topk_topp_sampler.py:92-139``)."""
    if top_k is None and top_p is None:
        return logits
    srt, idx = logits.float().sort(-1, descending=False)
    V = logits.shape[-1]
    if top_k is not None:
        k = top_k.long().clamp(1, V)
        thresh = srt.gather(1, (V - k).unsqueeze(1))
        srt = srt.masked_fill(srt < thresh, float("-inf"))
    if top_p is not None:
        probs = srt.softmax(-1)
        cum = probs.cumsum(-1)
        mask = cum <= (1 - top_p.float()).unsqueeze(1)
        mask[:, -1] = False
        srt = srt.masked_fill(mask, float("-inf"))
    return torch.empty_like(srt).scatter_(-1, idx, srt)


def random_sample(probs, generator=None, q: Optional[torch.Tensor] = None):
    """Exponential-race sampling (``topk_topp_sampler.py:141-174``): ``argmax(p / Exp(1))``."""
    if q is None:
        q = torch.empty_like(probs).exponential_(generator=generator)
    return (probs / q).argmax(-1)


def sample(logits, temperature, top_k=None, top_p=None, generator=None, q=None):
    """Greedy where ``temperature == 0``; otherwise temperature -> top-k/top-p -> softmax -> sample."""
    greedy = logits.float().argmax(-1)
    t = temperature.float()
    if bool((t == 0).all()):
        return greedy
    lg = logits.float() / torch.where(t == 0, torch.ones_like(t), t).unsqueeze(1)
    lg = apply_top_k_top_p(lg, top_k, top_p)
    rnd = random_sample(lg.softmax(-1), generator, q)
    return torch.where(t == 0, greedy, rnd)


def rejection_sample(draft_token_ids, cu_num_draft, draft_probs, target_probs, bonus_token_ids,
                     is_greedy, uniform=None, recover_q=None, max_spec_len: Optional[int] = None):
    """Speculative-decoding verifier (``v1/sample/rejection_sampler.py:134-641``).

    ``draft_token_ids [n]`` flattened over requests (``cu_num_draft [B+1]``), ``target_probs [n, V]``
    (for greedy rows only its argmax matters), ``draft_probs [n, V]`` or None (n-gram / greedy
    draft: probability 1), ``bonus_token_ids [B]``.  Output ``[B, max_spec_len+1]`` padded with -1.
    """
    B = bonus_token_ids.shape[0]
    nd = (cu_num_draft[1:] - cu_num_draft[:-1]).tolist()
    S = max_spec_len if max_spec_len is not None else max(nd + [0])
    out = torch.full((B, S + 1), PLACEHOLDER_TOKEN_ID, dtype=torch.int64)
    tgt_argmax = target_probs.argmax(-1)
    for b in range(B):
        st = int(cu_num_draft[b])
        rejected = False
        for j in range(nd[b]):
            tok = int(draft_token_ids[st + j])
            if bool(is_greedy[b]):
                t = int(tgt_argmax[st + j])
                out[b, j] = t
                if t != tok:
                    rejected = True
                    break
            else:
                dp = 1.0 if draft_probs is None else float(draft_probs[st + j, tok])
                tp = float(target_probs[st + j, tok])
                u = float(uniform[st + j])
                if dp > 0 and tp / dp >= u:
                    out[b, j] = tok
                else:
                    rejected = True
                    if draft_probs is None:
                        adj = target_probs[st + j].float().clone()
                        adj[tok] = 0
                    else:
                        adj = (target_probs[st + j].float() - draft_probs[st + j].float()).clamp(min=0)
                    q = recover_q[b].float() if recover_q is not None else torch.ones_like(adj)
                    out[b, j] = int((adj / q).argmax())
                    break
        if not rejected:
            out[b, nd[b]] = int(bonus_token_ids[b])
    return out


# ----------------------------------------------------------------------------- conv / GDN

def causal_conv1d_fn(x, weight, bias, cu_seqlens, conv_states, state_indices, has_initial_state,
                     activation: bool = True):
    """``kunlun_ops.causal_conv1d_fn`` (``ops/mamba/causal_conv1d.py:15-74``): varlen depthwise causal
    conv with a per-sequence state cache.  ``x [T, C]``, ``weight [C, W]``,
    ``conv_states [slots, W-1, C]`` (updated in place with the last ``W-1`` inputs)."""
    W = weight.shape[1]
    out = torch.empty_like(x)
    for r in range(len(cu_seqlens) - 1):
        s, e = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        if e == s:
            continue
        slot = int(state_indices[r])
        init = conv_states[slot].float() if bool(has_initial_state[r]) else torch.zeros(W - 1, x.shape[1])
        seq = torch.cat([init, x[s:e].float()], 0)  # [W-1+L, C]
        win = seq.unfold(0, W, 1)  # [L, C, W]
        y = (win * weight.float().unsqueeze(0)).sum(-1)
        if bias is not None:
            y = y + bias.float()
        if activation:
            y = torch.nn.functional.silu(y)
        out[s:e] = y.to(x.dtype)
        conv_states[slot] = seq[-(W - 1):].to(conv_states.dtype)
    return out


def causal_conv1d_update(x, conv_states, weight, bias, state_indices, activation: bool = True):
    """``kunlun_ops.causal_conv1d_update`` (``ops/mamba/causal_conv1d.py:118-225``): one token per
    sequence.  ``x [B, C]``."""
    out = torch.empty_like(x)
    for b in range(x.shape[0]):
        slot = int(state_indices[b])
        if slot < 0:
            out[b] = 0
            continue
        seq = torch.cat([conv_states[slot].float(), x[b:b + 1].float()], 0)  # [W, C]
        y = (seq.T * weight.float()).sum(-1)
        if bias is not None:
            y = y + bias.float()
        if activation:
            y = torch.nn.functional.silu(y)
        out[b] = y.to(x.dtype)
        conv_states[slot] = seq[1:].to(conv_states.dtype)
    return out


def recurrent_gated_delta_rule(q, k, v, g, beta, state, scale: Optional[float] = None,
                               use_qk_l2norm: bool = True):
    """Token-by-token gated delta rule (``ops/fla/fused_recurrent.py:52-155``).
    ``q, k [L, Hk, Dk]``, ``v [L, Hv, Dv]``, ``g, beta [L, Hv]``, ``state [Hv, Dv, Dk]``.
    ``S <- S * exp(g); S += beta * (v - S k) k^T; o = S q``.  Returns ``(o [L, Hv, Dv], state)``."""
    L, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf, kf = q.float(), k.float()
    if use_qk_l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = qf.repeat_interleave(rep, 1) * (scale if scale is not None else Dk ** -0.5)
    kf = kf.repeat_interleave(rep, 1)
    S = state.float().clone()
    out = torch.empty(L, Hv, Dv)
    for t in range(L):
        S = S * torch.exp(g[t].float()).reshape(Hv, 1, 1)
        pred = torch.einsum("hvk,hk->hv", S, kf[t])
        delta = (v[t].float() - pred) * beta[t].float().unsqueeze(-1)
        S = S + torch.einsum("hv,hk->hvk", delta, kf[t])
        out[t] = torch.einsum("hvk,hk->hv", S, qf[t])
    return out.to(v.dtype), S


def chunk_gated_delta_rule(q, k, v, g, beta, state, chunk: int = 64, scale=None, use_qk_l2norm=True):
    """Chunked (prefill) form of the gated delta rule (``ops/fla/chunk.py:23-140``: local cumsum,
    scaled ``K K^T``, triangular solve, ``w/u`` recompute, inter-chunk state, output).  Numerically
    equal to the recurrent form; used to validate the chunked kernels."""
    L, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf, kf = q.float(), k.float()
    if use_qk_l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = (qf.repeat_interleave(rep, 1) * (scale if scale is not None else Dk ** -0.5)).permute(1, 0, 2)
    kf = kf.repeat_interleave(rep, 1).permute(1, 0, 2)  # [Hv, L, Dk]
    vf = v.float().permute(1, 0, 2)
    gf = g.float().T  # [Hv, L]
    bf = beta.float().T
    S = state.float().clone()  # [Hv, Dv, Dk]
    out = torch.empty(Hv, L, Dv)
    for c0 in range(0, L, chunk):
        c1 = min(c0 + chunk, L)
        n = c1 - c0
        qc, kc, vc = qf[:, c0:c1], kf[:, c0:c1], vf[:, c0:c1]
        gc = gf[:, c0:c1].cumsum(-1)  # local cumulative log decay
        bc = bf[:, c0:c1]
        decay = torch.exp(gc.unsqueeze(-1) - gc.unsqueeze(-2))  # [Hv, n, n] exp(g_i - g_j)
        tril_strict = torch.tril(torch.ones(n, n), -1).bool()
        A = (kc @ kc.transpose(-1, -2)) * decay * bc.unsqueeze(-1)
        A = A.masked_fill(~tril_strict, 0)
        Tm = torch.linalg.solve_triangular(torch.eye(n) + A, torch.eye(n).expand(Hv, n, n).clone(), upper=False)
        u = Tm @ (vc * bc.unsqueeze(-1))
        w = Tm @ (kc * (bc * torch.exp(gc)).unsqueeze(-1))
        v_new = u - w @ S.transpose(-1, -2)  # [Hv, n, Dv]
        attn = (qc @ kc.transpose(-1, -2)) * decay
        attn = attn.masked_fill(~torch.tril(torch.ones(n, n)).bool(), 0)
        out[:, c0:c1] = (qc * torch.exp(gc).unsqueeze(-1)) @ S.transpose(-1, -2) + attn @ v_new
        glast = gc[:, -1]
        kdec = kc * torch.exp(glast.unsqueeze(-1) - gc).unsqueeze(-1)
        S = S * torch.exp(glast).reshape(Hv, 1, 1) + v_new.transpose(-1, -2) @ kdec
    return out.permute(1, 0, 2).to(v.dtype), S


def chunk_gated_delta_rule_batched(q, k, v, g, beta, state, chunk: int = 64, scale=None, use_qk_l2norm=True):
    """The chunked form with everything that does not depend on the running state computed for ALL chunks at once
    (decays, the unit-lower-triangular solve, ``u`` / ``w``, the intra-chunk attention: batched matrix products on the
    tensors' own device), followed by one short loop over the chunks that carries the state - three small products
    per chunk instead of one dependent step per token.  The sequence is padded to a multiple of ``chunk`` with steps
    that change nothing (``g = 0``, ``beta = 0``).  Same arguments and results as
    :func:`recurrent_gated_delta_rule`; fp32 inside."""
    L, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    rep, dev = Hv // Hk, q.device
    qf, kf = q.float(), k.float()
    if use_qk_l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = qf * (scale if scale is not None else Dk ** -0.5)
    pad = (-L) % chunk
    N = (L + pad) // chunk

    def blocks(x, heads_from_k):            # [L, H, D] -> [Hv, N, chunk, D]
        if pad:
            x = torch.cat([x, x.new_zeros(pad, *x.shape[1:])])
        if heads_from_k and rep > 1:
            x = x.repeat_interleave(rep, 1)
        return x.permute(1, 0, 2).reshape(Hv, N, chunk, x.shape[-1])

    qc, kc, vc = blocks(qf, True), blocks(kf, True), blocks(v.float(), False)
    gc = blocks(g.float().unsqueeze(-1), False).squeeze(-1).cumsum(-1)        # [Hv, N, chunk] log decay inside a chunk
    bc = blocks(beta.float().unsqueeze(-1), False).squeeze(-1)
    lower = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=dev))
    diff = gc.unsqueeze(-1) - gc.unsqueeze(-2)                                  # g_i - g_j
    decay = torch.exp(diff.masked_fill(~lower, float("-inf")))                  # 0 above the diagonal
    kk = kc @ kc.transpose(-1, -2)
    eye = torch.eye(chunk, device=dev)
    A = kk * decay * bc.unsqueeze(-1) * (~eye.bool())                           # strictly lower
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand(Hv, N, chunk, chunk).contiguous(), upper=False)
    u = Tm @ (vc * bc.unsqueeze(-1))
    w = Tm @ (kc * (bc * torch.exp(gc)).unsqueeze(-1))
    attn = (qc @ kc.transpose(-1, -2)) * decay
    qg = qc * torch.exp(gc).unsqueeze(-1)
    glast = gc[..., -1]
    kdec = kc * torch.exp(glast.unsqueeze(-1) - gc).unsqueeze(-1)
    eg = torch.exp(glast)
    S = state.float().clone()                                                   # [Hv, Dv, Dk]
    out = torch.empty(Hv, N, chunk, Dv, dtype=torch.float32, device=dev)
    for n in range(N):
        St = S.transpose(-1, -2)
        v_new = u[:, n] - w[:, n] @ St
        out[:, n] = qg[:, n] @ St + attn[:, n] @ v_new
        S = S * eg[:, n].reshape(Hv, 1, 1) + v_new.transpose(-1, -2) @ kdec[:, n]
    return out.reshape(Hv, N * chunk, Dv)[:, :L].permute(1, 0, 2).to(v.dtype), S


# ----------------------------------------------------------------------------- LoRA

def sgmv_shrink(x, lora_a, seq_lod, lora_ids, scale: float):
    """``_C::sgmv_shrink_lora`` (``ops/_custom_ops.py:2435-2519``): per-segment ``x @ A[id].T * scale``.
    ``lora_a [L, r, K]``; id < 0 = no adapter (zeros)."""
    out = torch.zeros(x.shape[0], lora_a.shape[1], dtype=torch.float32)
    for i, lid in enumerate(lora_ids.tolist()):
        s, e = int(seq_lod[i]), int(seq_lod[i + 1])
        if lid >= 0 and e > s:
            out[s:e] = x[s:e].float() @ lora_a[lid].float().T * scale
    return out


def sgmv_expand(h, lora_b, seq_lod, lora_ids, out, offset: int = 0, add: bool = True):
    """``_C::sgmv_expand(_slice)_lora`` (``ops/_custom_ops.py:2520-2676``): ``out[:, off:off+N] (+)= h @ B[id].T``."""
    N = lora_b.shape[1]
    for i, lid in enumerate(lora_ids.tolist()):
        s, e = int(seq_lod[i]), int(seq_lod[i + 1])
        if lid >= 0 and e > s:
            y = (h[s:e].float() @ lora_b[lid].float().T).to(out.dtype)
            if add:
                out[s:e, offset:offset + N] += y
            else:
                out[s:e, offset:offset + N] = y
    return out


def bgmv_shrink(x, lora_a, token_ids, scale: float):
    """``_C::bgmv_shrink_lora`` (``ops/_custom_ops.py:2677-2730``): per-token adapter."""
    out = torch.zeros(x.shape[0], lora_a.shape[1], dtype=torch.float32)
    for t, lid in enumerate(token_ids.tolist()):
        if lid >= 0:
            out[t] = x[t].float() @ lora_a[lid].float().T * scale
    return out


def bgmv_expand(h, lora_b, token_ids, out, offset: int = 0, add: bool = True):
    """``_C::bgmv_expand(_slice)_lora`` (``ops/_custom_ops.py:2731-2836``)."""
    N = lora_b.shape[1]
    for t, lid in enumerate(token_ids.tolist()):
        if lid >= 0:
            y = (h[t].float() @ lora_b[lid].float().T).to(out.dtype)
            if add:
                out[t, offset:offset + N] += y
            else:
                out[t, offset:offset + N] = y
    return out
