"""CUDA kernels vs the fp32 PyTorch oracles (run with ``-m gpu`` on a B200)."""
import math

import pytest
import torch

from vllm_kunlun_b200 import ops
from vllm_kunlun_b200.ops.reference import attention as ra
from vllm_kunlun_b200.ops.reference import basic as rb

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, name=""):
    """Every element must meet ``|a - b| <= atol + rtol * |b|`` (no outlier allowance: a wrong row at a tile edge
    is a failure)."""
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape, f"{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{name}: non-finite output"
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{name}: {int(bad.sum())} of {bad.numel()} elements off, max err "
                             f"{err.max().item():.4g}, first at {idx}: {a[tuple(idx)].item():.5g} vs "
                             f"{b[tuple(idx)].item():.5g}")


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 4096, 4096), (17, 384, 512), (64, 200, 256),
                                   (200, 1024, 1024), (512, 2048, 768), (1000, 640, 4096), (16, 6144, 4096),
                                   (16, 4096, 14336), (3, 128256 // 8, 512)])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_gemm_bf16(T, N, K, splits):
    from vllm_kunlun_b200.ops.gemm_cuda import check_status, gemm_bf16
    g = torch.Generator(device=DEV).manual_seed(T * 7 + N + K)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device=DEV, generator=g).to(torch.bfloat16)
    y = gemm_bf16(x, w, b, splits=splits)
    torch.cuda.synchronize()
    check_status()
    ref = x.float() @ w.float().T + b.float()
    _close(y, ref, atol=0.02 * math.sqrt(K / 64), rtol=0.02, name=f"gemm {T}x{N}x{K}/{splits}")


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (7, 768, 4096), (16, 4096, 512), (16, 4096, 1792), (16, 3584, 4096),
                                   (16, 1000, 200), (17, 640, 4096), (32, 4096, 4096), (30, 256, 14336)])
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 5, 8])
def test_gemm_decode_cluster_splitk(T, N, K, splits):
    """Cluster split-K decode kernel vs the fp32 oracle: every cluster size, ragged N / K, both token tiles."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    g = torch.Generator(device=DEV).manual_seed(T * 7 + N + K)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device=DEV, generator=g).to(torch.bfloat16)
    y = torch.full((T, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    _ext.C().gemm_decode(y, x, w, b, splits, 0, 0, 0)
    torch.cuda.synchronize()
    check_status()
    ref = x.float() @ w.float().T + b.float()
    # fp32 accumulation; the only rounding is the bf16 output (2^-9 relative) and the order of the K sum
    _close(y, ref, atol=2e-3 * math.sqrt(K / 64), rtol=6e-3, name=f"gemm_decode {T}x{N}x{K}/{splits}")
    y2 = torch.empty_like(y)
    _ext.C().gemm_decode(y2, x, w, b, splits, 0, 0, 0)
    assert torch.equal(y, y2), "cluster split-K must be deterministic"


@pytest.mark.parametrize("T", [3, 16, 32])
@pytest.mark.parametrize("splits", [0, 1, 4])
def test_gemm_decode_gated_activation(T, splits):
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status, interleave_gate_up
    K, inter = 1024, 768
    g = torch.Generator(device=DEV).manual_seed(T)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    y = torch.empty(T, inter, device=DEV, dtype=torch.bfloat16)
    _ext.C().gemm_decode(y, x, interleave_gate_up(w), None, splits, 0, 0, 1)
    torch.cuda.synchronize()
    check_status()
    gu = (x.float() @ w.float().T).to(torch.bfloat16).float()  # the unfused path rounds the projection first
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    _close(y, ref, atol=0.02, rtol=0.02, name=f"gemm_decode silu {T}/{splits}")


def test_gemm_fp16_strided_out():
    from vllm_kunlun_b200.ops.gemm_cuda import check_status, gemm_bf16
    x = torch.randn(40, 320, device=DEV).half()
    w = (torch.randn(256, 320, device=DEV) * 0.05).half()
    y = gemm_bf16(x, w)
    torch.cuda.synchronize()
    check_status()
    _close(y, x.float() @ w.float().T, 0.03, 0.02, "gemm fp16")


def test_gemm_deterministic():
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_bf16
    x = torch.randn(16, 4096, device=DEV).bfloat16()
    w = (torch.randn(4096, 4096, device=DEV) * 0.02).bfloat16()
    a = gemm_bf16(x, w, splits=4).clone()
    for _ in range(3):
        assert torch.equal(a, gemm_bf16(x, w, splits=4))


@pytest.mark.parametrize("T,H", [(1, 896), (16, 4096), (33, 7168), (5, 16384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rmsnorm(T, H, dtype):
    x = torch.randn(T, H, device=DEV).to(dtype)
    r = torch.randn(T, H, device=DEV).to(dtype)
    w = torch.randn(H, device=DEV).to(dtype)
    _close(ops.rmsnorm(x, w, 1e-5), rb.rmsnorm(x.cpu(), w.cpu(), 1e-5), 1e-2, 1e-2, "rmsnorm")
    eo, er = rb.add_rmsnorm(x.cpu(), r.cpu(), w.cpu(), 1e-5)
    xo, ro = ops.add_rmsnorm(x.clone(), r.clone(), w, 1e-5)
    _close(xo, eo, 2e-2, 2e-2, "add_rmsnorm out")
    _close(ro, er, 1e-2, 1e-2, "add_rmsnorm residual")
    _close(ops.rmsnorm(x, w, 1e-6, gemma=True), rb.rmsnorm(x.cpu(), w.cpu(), 1e-6, True), 2e-2, 2e-2, "gemma")


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "swigluoai"])
def test_act_and_mul(act):
    x = torch.randn(19, 2 * 1536, device=DEV).bfloat16()
    ref = {"silu": rb.silu_and_mul, "gelu_tanh": rb.gelu_tanh_and_mul, "swigluoai": rb.swigluoai_and_mul}[act](x.cpu())
    _close(ops.act_and_mul(x, act), ref, 2e-2, 2e-2, act)


def test_rownorm_variants():
    x = torch.randn(7, 12, 128, device=DEV).bfloat16()
    z = torch.randn(7, 12, 128, device=DEV).bfloat16()
    w = torch.randn(128, device=DEV).bfloat16()
    _close(ops.l2norm(x), rb.l2norm(x.cpu()), 1e-2, 1e-2, "l2norm")
    for nbg in (True, False):
        _close(ops.rms_norm_gated(x, z, w, 1e-6, nbg), rb.rms_norm_gated(x.cpu(), z.cpu(), w.cpu(), 1e-6, nbg),
               3e-2, 3e-2, f"gated {nbg}")
    _close(ops.quick_gelu(x), rb.quick_gelu(x.cpu()), 1e-2, 1e-2, "quick_gelu")


def test_embedding_argmax():
    w = torch.randn(1000, 256, device=DEV).bfloat16()
    ids = torch.tensor([0, 5, 999, 1200, 400], device=DEV)
    out = ops.embedding(ids, w, 0)
    assert torch.equal(out[:3], w[ids[:3]]) and out[3].abs().sum() == 0
    out2 = ops.embedding(ids, w[400:], 400)
    assert torch.equal(out2[2], w[999]) and out2[0].abs().sum() == 0 and torch.equal(out2[4], w[400])
    lg = torch.randn(9, 151936, device=DEV).bfloat16()
    assert torch.equal(ops.argmax(lg).cpu(), lg.float().argmax(-1).cpu())
    lg32 = torch.randn(3, 1000, device=DEV)
    assert torch.equal(ops.argmax(lg32), lg32.argmax(-1))


@pytest.mark.parametrize("qk_norm,neox,D", [(False, True, 128), (True, True, 128), (False, False, 64), (True, True, 64)])
def test_qkv_split_norm_rope_cache(qk_norm, neox, D):
    T, Hq, Hkv, bs, nblk = 23, 8, 2, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (T,), device=DEV)
    cs = rb.build_cos_sin_cache(D, 512, 10000.0).to(DEV)
    qw = torch.randn(D, device=DEV).bfloat16() if qk_norm else None
    kw = torch.randn(D, device=DEV).bfloat16() if qk_norm else None
    slots = torch.randperm(bs * nblk, device=DEV)[:T]
    slots[3] = -1
    cache = torch.zeros(nblk, 2, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
    q = ops.qkv_split_norm_rope_cache(qkv, pos, cs, qw, kw, 1e-6, Hq, Hkv, D, neox, cache, slots)
    cache_ref = torch.zeros(nblk, 2, Hkv, bs, D, dtype=torch.bfloat16)
    q_ref = ops.qkv_split_norm_rope_cache(qkv.cpu(), pos.cpu(), cs.cpu(), None if qw is None else qw.cpu(),
                                          None if kw is None else kw.cpu(), 1e-6, Hq, Hkv, D, neox, cache_ref, slots.cpu())
    _close(q, q_ref, 3e-2, 3e-2, "q")
    _close(cache, cache_ref, 3e-2, 3e-2, "cache")


def _make_paged(B, seq_lens, Hkv, D, bs, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed)
    max_blocks = max(-(-s // bs) for s in seq_lens) + 1
    nblk = sum(-(-s // bs) for s in seq_lens) + 3
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    k = 0
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = perm[k:k + n]
        k += n
    cache = (torch.randn(nblk, 2, Hkv, bs, D, generator=g) * 0.5).to(dtype)
    return cache, bt


@pytest.mark.parametrize("D,Hq,Hkv,bs", [(128, 32, 8, 16), (128, 8, 1, 64), (64, 14, 2, 16), (128, 16, 16, 32)])
@pytest.mark.parametrize("q_len", [1, 2])
def test_paged_attention_decode(D, Hq, Hkv, bs, q_len):
    seq_lens = [1 + q_len, 17, 64, 65, 300, 1000, 2049]
    B = len(seq_lens)
    cache, bt = _make_paged(B, seq_lens, Hkv, D, bs)
    qsl = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32)
    q = (torch.randn(B * q_len, Hq, D) * 0.5).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    scale = D ** -0.5
    ref = ra.paged_attention(q, cache, bt, sl, qsl, scale)
    for splits in (None, 1, 5):
        from vllm_kunlun_b200.ops.attention_cuda import paged_attention_cuda
        out = torch.empty(B * q_len, Hq, D, device=DEV, dtype=torch.bfloat16)
        paged_attention_cuda(out, q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), scale, q_len,
                             max(seq_lens), num_splits=splits)
        _close(out, ref, 2e-2, 2e-2, f"decode splits={splits}")


@pytest.mark.parametrize("D,Hq,Hkv,bs", [(128, 8, 2, 16), (64, 4, 4, 64), (128, 4, 1, 32)])
def test_paged_attention_prefill(D, Hq, Hkv, bs):
    # (q_len, seq_len): fresh prompts, chunked continuation with cached prefix, one decode row mixed in
    spec = [(1, 40), (37, 37), (128, 128), (70, 200), (300, 300), (5, 133)]
    B = len(spec)
    seq_lens = [s for _, s in spec]
    cache, bt = _make_paged(B, seq_lens, Hkv, D, bs, seed=1)
    qsl = torch.tensor([0] + list(torch.tensor([q for q, _ in spec]).cumsum(0)), dtype=torch.int32)
    T = int(qsl[-1])
    q = (torch.randn(T, Hq, D) * 0.5).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    scale = D ** -0.5
    ref = ra.paged_attention(q, cache, bt, sl, qsl, scale)
    out = ops.paged_attention(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), scale,
                              max(qq for qq, _ in spec), max(seq_lens), num_decodes=1)
    _close(out, ref, 2e-2, 2e-2, "prefill")


def test_paged_attention_window_sinks():
    D, Hq, Hkv, bs = 64, 8, 2, 16
    spec = [(1, 300), (1, 100), (150, 150), (40, 260)]
    B = len(spec)
    seq_lens = [s for _, s in spec]
    cache, bt = _make_paged(B, seq_lens, Hkv, D, bs, seed=2)
    qsl = torch.tensor([0] + list(torch.tensor([q for q, _ in spec]).cumsum(0)), dtype=torch.int32)
    q = (torch.randn(int(qsl[-1]), Hq, D) * 0.5).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    sinks = torch.randn(Hq)
    ref = ra.paged_attention(q, cache, bt, sl, qsl, 0.125, window=128, sinks=sinks)
    out = ops.paged_attention(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), 0.125, 150, 300,
                              window=128, sinks=sinks.to(DEV), num_decodes=2)
    _close(out, ref, 2e-2, 2e-2, "window+sinks")


def test_cache_ops():
    T, bs, nblk = 11, 64, 4
    kvc = torch.randn(T, 512, device=DEV).bfloat16()
    kpe = torch.randn(T, 64, device=DEV).bfloat16()
    slots = torch.randperm(bs * nblk, device=DEV)[:T]
    cache = torch.zeros(nblk, bs, 576, device=DEV, dtype=torch.bfloat16)
    ops.concat_and_cache_mla(kvc, kpe, cache, slots)
    ref = torch.zeros(nblk, bs, 576, dtype=torch.bfloat16)
    ra.concat_and_cache_mla(kvc.cpu(), kpe.cpu(), ref, slots.cpu())
    assert torch.equal(cache.cpu(), ref)
    c8 = torch.zeros(nblk, bs, 656, device=DEV, dtype=torch.uint8)
    ops.concat_and_cache_mla(kvc, kpe, c8, slots)
    r8 = torch.zeros(nblk, bs, 656, dtype=torch.uint8)
    ra.concat_and_cache_mla_fp8(kvc.cpu(), kpe.cpu(), r8, slots.cpu())
    _close(ra.dequant_mla_fp8_rows(c8.cpu()), ra.dequant_mla_fp8_rows(r8), 0.08, 0.08, "fp8_ds_mla")
    k = torch.randn(T, 128, device=DEV).bfloat16()
    ck = torch.zeros(nblk, bs, 132, device=DEV, dtype=torch.uint8)
    ops.indexer_k_quant_and_cache(k, ck, slots)
    rk = torch.zeros(nblk, bs, 132, dtype=torch.uint8)
    ra.indexer_k_quant_and_cache(k.cpu(), rk, slots.cpu())
    (ka, sa), (kb, sb) = ra.indexer_cache_views(ck.cpu()), ra.indexer_cache_views(rk)
    assert torch.equal(sa, sb)
    a = ka.contiguous().view(torch.float8_e4m3fn).float()
    b = kb.contiguous().view(torch.float8_e4m3fn).float()
    assert (a - b).abs().max() <= 32  # at most one e4m3 step apart
    idx = torch.randint(-1, 200, (T, 64), device=DEV, dtype=torch.int32)
    req = torch.randint(0, 3, (T,), device=DEV, dtype=torch.int32)
    btab = torch.randint(0, 50, (3, 4), device=DEV, dtype=torch.int32)
    got = ops.convert_req_index_to_global_index(req, btab, idx, 64)
    want = ra.convert_req_index_to_global_index(req.cpu(), btab.cpu(), idx.cpu(), 64)
    assert torch.equal(got.cpu(), want)
    o1, o2 = torch.randn(5, 4, 128, device=DEV).bfloat16(), torch.randn(5, 4, 128, device=DEV).bfloat16()
    l1, l2 = torch.randn(5, 4, device=DEV), torch.randn(5, 4, device=DEV)
    l2[0, 0] = float("-inf")
    mo, ml = ops.merge_attn_states(o1, l1, o2, l2)
    ro, rl = ra.merge_attn_states(o1.cpu(), l1.cpu(), o2.cpu(), l2.cpu())
    _close(mo, ro, 2e-2, 2e-2, "merge o")
    _close(ml, rl, 1e-3, 1e-3, "merge lse")


@pytest.mark.parametrize("Hq,Hkv,q_len", [(32, 8, 1), (4, 1, 1), (8, 2, 2), (16, 1, 1), (4, 4, 3)])
@pytest.mark.parametrize("splits", [None, 1, 3, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_attention_umma(Hq, Hkv, q_len, splits, dtype):
    """tcgen05 decode attention (keys on the UMMA M side) vs the fp32 oracle: ragged lengths that end inside a tile,
    inside a page and on a page edge, an empty request, several query tokens per request, split-KV merge."""
    from vllm_kunlun_b200.ops.attention_cuda import UMMA_DECODE, paged_attention_cuda
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    assert UMMA_DECODE[0]
    D, bs = 128, 64
    lens = [1, 63, 64, 65, 128, 129, 700, 1337, 5, 2048]
    lens = [max(n, q_len) for n in lens]
    B = len(lens)
    g = torch.Generator(device=DEV).manual_seed(Hq * 100 + q_len)
    nblk_per = [-(-n // bs) for n in lens]
    nblk = sum(nblk_per) + 3
    kv = (torch.randn(nblk, 2, Hkv, bs, D, device=DEV, generator=g) * 1.0).to(dtype)
    perm = torch.randperm(nblk - 1, device=DEV, generator=g) + 1  # block 0 stays unused
    bt = torch.zeros(B, max(nblk_per), dtype=torch.int32, device=DEV)
    o = 0
    for b, n in enumerate(nblk_per):
        bt[b, :n] = perm[o:o + n].int()
        o += n
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    qsl = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32, device=DEV)
    T = B * q_len
    q = torch.randn(T, Hq, D, device=DEV, generator=g).to(dtype)
    out = torch.full((T, Hq, D), float("nan"), device=DEV, dtype=dtype)
    scale = D ** -0.5
    paged_attention_cuda(out, q, kv, bt, seq_lens, qsl, scale, q_len, max(lens), None, None, None, splits)
    torch.cuda.synchronize()
    check_status()
    ref = ra.paged_attention(q.cpu(), kv.cpu(), bt.cpu(), seq_lens.cpu(), qsl.cpu(), scale, None, None)
    # P and V are 16-bit, sums are fp32: outputs are convex combinations of V rows of magnitude ~1
    _close(out, ref, atol=0.02, rtol=0.02, name=f"decode umma {Hq}/{Hkv}/{q_len}/{splits}")


def test_decode_attention_umma_window_and_sinks():
    from vllm_kunlun_b200.ops.attention_cuda import paged_attention_cuda
    D, bs, Hq, Hkv = 128, 64, 8, 2
    lens = [900, 131, 64, 300]
    B = len(lens)
    g = torch.Generator(device=DEV).manual_seed(3)
    nblk_per = [-(-n // bs) for n in lens]
    nblk = sum(nblk_per) + 1
    kv = torch.randn(nblk, 2, Hkv, bs, D, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.zeros(B, max(nblk_per), dtype=torch.int32, device=DEV)
    o = 1
    for b, n in enumerate(nblk_per):
        bt[b, :n] = torch.arange(o, o + n, dtype=torch.int32, device=DEV)
        o += n
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    qsl = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    q = torch.randn(B, Hq, D, device=DEV, generator=g).to(torch.bfloat16)
    sinks = torch.randn(Hq, device=DEV, generator=g)
    for window, sk, splits in [(200, None, 1), (200, sinks, 2), (None, sinks, 3)]:
        out = torch.empty(B, Hq, D, device=DEV, dtype=torch.bfloat16)
        paged_attention_cuda(out, q, kv, bt, seq_lens, qsl, D ** -0.5, 1, max(lens), window, sk, None, splits)
        ref = ra.paged_attention(q.cpu(), kv.cpu(), bt.cpu(), seq_lens.cpu(), qsl.cpu(), D ** -0.5, window,
                                 None if sk is None else sk.cpu())
        _close(out, ref, atol=0.02, rtol=0.02, name=f"decode umma window={window} sinks={sk is not None}")


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("T", [1, 16, 200, 1000])
def test_gemm_fused_gated_activation(T, act):
    """Gate/up projection with the activation in the GEMM epilogue == projection followed by act_and_mul (bitwise:
    the epilogue rounds gate and up to bf16 before the activation, exactly like the two-kernel path)."""
    from vllm_kunlun_b200.ops.gemm_cuda import gemm_bf16, interleave_gate_up
    torch.manual_seed(T)
    K, I = 512, 1536
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda") * 0.05).to(torch.bfloat16)
    b = (torch.randn(2 * I, device="cuda") * 0.1).to(torch.bfloat16)
    want = ops.act_and_mul(gemm_bf16(x, w, b, splits=1), act)  # whole tiles: the same fp32 summation order
    got = ops.linear_gated_act(x, interleave_gate_up(w), interleave_gate_up(b), act)
    assert got.shape == (T, I)
    if T > 32:
        assert torch.equal(got, want)
    else:  # decode-sized calls split K over a cluster whose size follows the tile count: another summation order
        _close(got, want, atol=0.01, rtol=0.02, name=f"fused {act} T={T}")
    ref = ops.act_and_mul((x.float().cpu() @ w.float().cpu().T + b.float().cpu()).to(torch.bfloat16), act)
    torch.testing.assert_close(got.float().cpu(), ref.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("T,Hq,Hkv,qk_norm,neox", [(16, 32, 8, False, True), (5, 4, 1, True, True), (32, 8, 2, True, False),
                                                    (1, 16, 2, False, False)])
def test_gemm_decode_qkv_epilogue(T, Hq, Hkv, qk_norm, neox):
    """Decode qkv projection with split + q / k RMSNorm + rotary + paged-cache write in its epilogue == the projection
    followed by the stand-alone split / norm / rope / cache kernel, bit for bit (both round the projection to bf16
    first; the K sum is taken in the same order because the cluster size follows the same rule)."""
    from vllm_kunlun_b200.models.layers import get_cos_sin_cache
    from vllm_kunlun_b200.ops import _ext, gemm_cuda
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    D, K, bs, nblk = 128, 1024, 64, 5
    g = torch.Generator(device=DEV).manual_seed(T + Hq)
    N = (Hq + 2 * Hkv) * D
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.04).bfloat16()
    b = (torch.randn(N, device=DEV, generator=g) * 0.1).bfloat16()
    qw = (torch.rand(D, device=DEV, generator=g) + 0.5).bfloat16() if qk_norm else None
    kw = (torch.rand(D, device=DEV, generator=g) + 0.5).bfloat16() if qk_norm else None
    pos = torch.randint(0, 3000, (T,), device=DEV, generator=g)
    slots = torch.randperm(nblk * bs, device=DEV, generator=g)[:T].long()
    if T > 2:
        slots[2] = -1
    cos_sin = get_cos_sin_cache(D, 4096, 10000.0, None, DEV)
    cache = torch.zeros(nblk, 2, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
    q = gemm_cuda.gemm_decode_qkv(x, w, b, pos, cos_sin, qw, kw, 1e-6, Hq, Hkv, neox, False, cache, slots)
    torch.cuda.synchronize()
    check_status()
    qkv = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    _ext.C().gemm_decode(qkv, x, w, b, 0, 0, 0, 0)
    cache2 = torch.zeros_like(cache)
    q2 = ops.qkv_split_norm_rope_cache(qkv, pos, cos_sin, qw, kw, 1e-6, Hq, Hkv, D, neox, cache2, slots)
    torch.cuda.synchronize()
    assert torch.equal(q, q2)
    assert torch.equal(cache, cache2)
    # and against fp32 arithmetic on the rounded projection
    from vllm_kunlun_b200.ops.reference import basic as rb
    ref_qkv = (x.float().cpu() @ w.float().cpu().T + b.float().cpu()).bfloat16()
    rq, rk, rv = rb.split_qknorm_rope(ref_qkv, pos.cpu(), cos_sin.cpu(), None if qw is None else qw.cpu(),
                                      None if kw is None else kw.cpu(), 1e-6, Hq, Hkv, D, neox, False)
    _close(q, rq, atol=0.06, rtol=0.03, name="qkv epilogue q")


@pytest.mark.parametrize("T,N,K", [(16, 512, 1024), (1, 128, 256), (32, 1000, 4096), (100, 384, 2048), (300, 1536, 7168),
                                   (7, 2048, 11008 // 16 * 16)])
@pytest.mark.parametrize("static", [False, True])
def test_int8_w8a8_tensor_core_gemm(T, N, K, static):
    """W8A8 int8 on tcgen05 kind::i8 (s32 accumulation: exact integer sums) - the activation quantiser, the cluster
    split-K kernel (<= 32 rows) and the dense kernel - against integer arithmetic on the same quantised operands."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    from vllm_kunlun_b200.ops.reference import basic as rb
    g = torch.Generator().manual_seed(T + N)
    x = (torch.randn(T, K, generator=g) * 1.5).bfloat16()
    wf = torch.randn(N, K, generator=g) * 0.05
    ws = wf.abs().amax(-1, keepdim=True).clamp(min=1e-8) / 127.0
    wq = torch.round(wf / ws).clamp(-128, 127).to(torch.int8)
    bias = torch.randn(N, generator=g).bfloat16()
    in_scale = torch.tensor([0.04]) if static else None
    C = _ext.C()
    q, s = C.quant_int8_token(x.to(DEV), None if in_scale is None else in_scale.to(DEV))
    if static:
        rq, rs = rb.quant_int8_static(x, in_scale), in_scale.expand(T).reshape(T, 1)
    else:
        rq, rs = rb.quant_int8_per_token(x)
    torch.testing.assert_close(s.cpu(), rs.reshape(-1).float(), rtol=1e-6, atol=0)
    assert (q.cpu().int() - rq.int()).abs().max() <= 1        # a value on a rounding edge may land on either side
    assert (q.cpu() != rq).float().mean() < 1e-3
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    C.gemm_int8(out, q, wq.to(DEV), bias.to(DEV), s, ws.reshape(-1).to(DEV))
    torch.cuda.synchronize()
    check_status()
    ref = rb.int8_scaled_mm(q.cpu(), s.cpu().reshape(T, 1), wq, ws.reshape(-1), bias, torch.float32)
    # integer sums are exact; what is left is the bf16 rounding of the output
    _close(out, ref, atol=1e-2, rtol=8e-3, name=f"int8 gemm {T}x{N}x{K}")
    # and through the functional entry point
    y = ops.int8_linear(x.to(DEV), wq.to(DEV), ws.to(DEV), bias.to(DEV), None if in_scale is None else in_scale.to(DEV))
    assert torch.equal(y, out)


@pytest.mark.parametrize("Hq,Hkv,bs", [(8, 2, 64), (4, 4, 128), (16, 1, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill_attention_umma(Hq, Hkv, bs, dtype):
    """tcgen05 prefill attention (128 query rows of one head per CTA, S and O in TMEM) vs the fp32 oracle: fresh
    prompts, chunked continuations over a cached prefix, lengths that end inside a tile / a page, a single-row
    request, more than one query tile per request; then a sliding window with sinks, and the log-sum-exp output."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.attention_cuda import UMMA_PREFILL, paged_attention_cuda
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    assert UMMA_PREFILL[0]
    D = 128
    spec = [(1, 40), (37, 37), (128, 128), (70, 200), (300, 300), (5, 133), (129, 1000), (450, 1500)]
    B = len(spec)
    seq_lens = [s for _, s in spec]
    cache, bt = _make_paged(B, seq_lens, Hkv, D, bs, dtype=dtype, seed=3)
    qsl = torch.tensor([0] + list(torch.tensor([q for q, _ in spec]).cumsum(0)), dtype=torch.int32)
    T = int(qsl[-1])
    q = (torch.randn(T, Hq, D, generator=torch.Generator().manual_seed(5)) * 0.5).to(dtype)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    scale = D ** -0.5
    mq = max(qq for qq, _ in spec)
    d = lambda x: x.to(DEV)
    ref = ra.paged_attention(q, cache, bt, sl, qsl, scale)
    out = torch.full((T, Hq, D), float("nan"), device=DEV, dtype=dtype)
    paged_attention_cuda(out, d(q), d(cache), d(bt), d(sl), d(qsl), scale, mq, max(seq_lens))
    torch.cuda.synchronize()
    check_status()
    _close(out, ref, 2e-2, 2e-2, "prefill umma")
    # sliding window + sinks
    sinks = torch.randn(Hq, generator=torch.Generator().manual_seed(6))
    ref_w = ra.paged_attention(q, cache, bt, sl, qsl, scale, 150, sinks)
    out_w = torch.full((T, Hq, D), float("nan"), device=DEV, dtype=dtype)
    paged_attention_cuda(out_w, d(q), d(cache), d(bt), d(sl), d(qsl), scale, mq, max(seq_lens), 150, d(sinks))
    torch.cuda.synchronize()
    check_status()
    _close(out_w, ref_w, 2e-2, 2e-2, "prefill umma window + sinks")
    # log-sum-exp (natural log) of every row
    lse = torch.full((T, Hq), float("nan"), device=DEV)
    out2 = torch.empty_like(out)
    _ext.C().prefill_attention_umma(out2, d(q), d(cache), d(bt), d(sl), d(qsl), None, lse, mq, 0, scale)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    want = []
    for b, (ql, s) in enumerate(spec):
        pos = torch.arange(s)
        k = cache[bt[b, pos // bs].long(), 0, :, pos % bs].float()          # [s, Hkv, D]
        g = Hq // Hkv
        for r in range(ql):
            qr = q[int(qsl[b]) + r].float()                                 # [Hq, D]
            n = s - ql + r + 1
            sc = torch.einsum("hd,nhd->hn", qr, k[:n].repeat_interleave(g, 1)) * scale
            want.append(torch.logsumexp(sc, -1))
    torch.testing.assert_close(lse.cpu(), torch.stack(want), atol=2e-2, rtol=2e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,K,group,splits", [(1, 256, 512, 128, 0), (16, 300, 1024, 64, 0), (16, 4096, 4096, 128, 0),
                                                (32, 1024, 2048, 128, 0), (5, 384, 4096, 128, 4), (16, 128, 4096, 4096, 8),
                                                (16, 6144, 4096, 128, 1)])
def test_gemm_decode_w4(dtype, T, N, K, group, splits):
    """Decode GEMM over 4-bit weights (packed bytes streamed by TMA, de-quantised by the epilogue warps into the
    swizzled A tile, then tcgen05): against the fp32 oracle over the de-quantised weight, and - with the same cluster
    size - bit for bit against the 16-bit decode GEMM over that weight (the kernel computes (q - zero) * scale with one
    rounding, as the oracle does).  Covers a partial last weight tile, groups of 64 / 128 / K, bias, both 16-bit types."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    from vllm_kunlun_b200.quantization.int4 import dequant_w4, pack_w4
    g = torch.Generator().manual_seed(T + N + K + group)
    q = torch.randint(0, 16, (N, K), generator=g)
    zero = torch.randint(0, 17, (N, K // group), generator=g).to(dtype)          # GPTQ's +1 convention reaches 16
    scale = (torch.rand(N, K // group, generator=g) * 0.02 + 0.005).to(dtype)
    packed = pack_w4(q)
    w = dequant_w4(packed, scale, zero, group)                                    # [N, K] in dtype
    x = torch.randn(T, K, generator=g).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype)
    C = _ext.C()
    pd, sd, zd, xd, bd = packed.to(DEV), scale.to(DEV), zero.to(DEV), x.to(DEV), bias.to(DEV)
    out = torch.empty(T, N, dtype=dtype, device=DEV)
    C.gemm_decode_w4(out, xd, pd, sd, zd, bd, group, splits, 0)
    check_status()
    want = x.float() @ w.float().T + bias.float()
    _close(out, want, 0.02 * math.sqrt(K / 512), 0.02, f"w4 decode {T}x{N}x{K} g{group}")
    # the de-quantising kernel for large batches: exact
    wd = torch.empty(N, K, dtype=dtype, device=DEV)
    C.dequant_w4(wd, pd, sd, zd, group)
    assert torch.equal(wd.cpu(), w)
    if splits > 0:   # same cluster size -> same sequence of MMAs and the same reduction order
        ref = torch.empty(T, N, dtype=dtype, device=DEV)
        C.gemm_decode(ref, xd, wd, bd, splits, 0, 0, 0)
        check_status()
        assert torch.equal(out, ref)
    # the op wrapper: decode-sized and larger batches
    y = ops.w4_linear(xd, pd, sd, zd, group, bd)
    if splits == 0:
        assert torch.equal(y, out)
    else:   # the wrapper lets the library choose the cluster size: another reduction order
        _close(y, want, 0.02 * math.sqrt(K / 512), 0.02, "w4 wrapper")
    xl = torch.randn(70, K, generator=g).to(dtype)
    yl = ops.w4_linear(xl.to(DEV), pd, sd, zd, group, bd)
    _close(yl, xl.float() @ w.float().T + bias.float(), 0.02 * math.sqrt(K / 512), 0.02, "w4 large batch")
