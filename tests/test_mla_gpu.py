"""MLA CUDA kernels (absorbed attention, dense and sparse; per-head products) vs the fp32 oracles."""
import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams, ops
from vllm_kunlun_b200.config import RopeScaling, deepseek_v3, tiny
from vllm_kunlun_b200.ops.reference import attention as ra

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, name=""):
    """Every element must meet ``|a - b| <= atol + rtol * |b|``."""
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape and torch.isfinite(a).all(), name
    err = (a - b).abs()
    bad = err > atol + rtol * b.abs()
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{name}: {int(bad.sum())} of {bad.numel()} elements off, max err {err.max().item():.4g}, "
                             f"first at {idx}: {a[tuple(idx)].item():.5g} vs {b[tuple(idx)].item():.5g}")


@pytest.mark.parametrize("N,q_len", [(16, 1), (16, 2), (5, 1), (128, 1), (40, 2), (8, 4)])
@pytest.mark.parametrize("splits", [None, 1, 2, 4, 8, 3, 16, -4])
def test_mla_decode_umma(N, q_len, splits):
    """tcgen05 MLA decode (cache pages as the UMMA M side, V = first 512 dims of the same shared-memory page) vs the
    fp32 oracle: lengths that end inside / on the edge of a page, several query tokens, head groups, split-KV merge
    inside a cluster (2 / 4 / 8 splits) and through the workspace (other counts; -4 = 4 splits forced that way)."""
    from vllm_kunlun_b200.ops import mla_cuda
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    from vllm_kunlun_b200.ops.mla_cuda import mla_decode_umma
    mla_cuda._FORCE_WORKSPACE[0] = splits is not None and splits < 0
    splits = abs(splits) if splits is not None else None
    bs = 64
    seq_lens = [q_len, 63 + q_len, 64, 65, 129, 700, 1500]
    B = len(seq_lens)
    g = torch.Generator().manual_seed(N * 10 + q_len)
    nblk = sum(-(-s // bs) for s in seq_lens) + 2
    perm = torch.randperm(nblk - 1, generator=g) + 1
    bt = torch.zeros(B, max(-(-s // bs) for s in seq_lens) + 1, dtype=torch.int32)
    k = 0
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = perm[k:k + n]
        k += n
    cache = (torch.randn(nblk, bs, 576, generator=g) * 0.3).bfloat16()
    q = (torch.randn(B * q_len, N, 576, generator=g) * 0.3).bfloat16()
    qsl = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    ref = ra.mla_decode(q, cache, bt, sl, qsl, 0.1)
    out = mla_decode_umma(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), 0.1, q_len, max(seq_lens), splits)
    torch.cuda.synchronize()
    mla_cuda._FORCE_WORKSPACE[0] = False
    check_status()
    _close(out, ref, 1e-2, 2e-2, f"mla umma N={N} q_len={q_len} splits={splits}")


@pytest.mark.parametrize("N", [16, 128, 5])
@pytest.mark.parametrize("q_len", [1, 2])
def test_mla_dense(N, q_len):
    bs = 64
    seq_lens = [q_len + 1, 33, 64, 65, 700, 2100]
    B = len(seq_lens)
    g = torch.Generator().manual_seed(N + q_len)
    nblk = sum(-(-s // bs) for s in seq_lens) + 2
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros(B, max(-(-s // bs) for s in seq_lens) + 1, dtype=torch.int32)
    k = 0
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = perm[k:k + n]
        k += n
    cache = (torch.randn(nblk, bs, 576, generator=g) * 0.3).bfloat16()
    q = (torch.randn(B * q_len, N, 576, generator=g) * 0.3).bfloat16()
    qsl = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    scale = 0.1
    ref = ra.mla_decode(q, cache, bt, sl, qsl, scale)
    out = ops.mla_attention(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), scale, 512, q_len,
                            max(seq_lens))
    _close(out, ref, 2e-2, 3e-2, f"mla dense N={N} q_len={q_len}")


def test_mla_prefill_rows():
    bs, N = 64, 16
    spec = [(40, 40), (100, 300), (1, 77)]
    g = torch.Generator().manual_seed(9)
    seq_lens = [s for _, s in spec]
    nblk = sum(-(-s // bs) for s in seq_lens) + 1
    bt = torch.zeros(len(spec), 6, dtype=torch.int32)
    k = 0
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = torch.arange(k, k + n)
        k += n
    cache = (torch.randn(nblk, bs, 576, generator=g) * 0.3).bfloat16()
    qsl = torch.tensor([0, 40, 140, 141], dtype=torch.int32)
    q = (torch.randn(141, N, 576, generator=g) * 0.3).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    ref = ra.mla_decode(q, cache, bt, sl, qsl, 0.1)
    out = ops.mla_attention(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), 0.1, 512, 100, 300)
    _close(out, ref, 2e-2, 3e-2, "mla prefill rows")


@pytest.mark.parametrize("topk", [64, 2048])
def test_sparse_mla(topk):
    g = torch.Generator().manual_seed(topk)
    T, N, slots = 9, 16, 5000
    cache = (torch.randn(slots // 64 + 1, 64, 576, generator=g) * 0.3).bfloat16()
    q = (torch.randn(T, N, 576, generator=g) * 0.3).bfloat16()
    idx = torch.full((T, topk), -1, dtype=torch.int32)
    for t in range(T):
        n = int(torch.randint(1, min(topk, slots) + 1, (1,), generator=g))
        idx[t, :n] = torch.randperm(slots, generator=g)[:n].to(torch.int32)
    idx[3, 5] = -1  # a hole in the middle of the list
    ref, _, _ = ra.sparse_mla(q, cache.reshape(-1, 576), idx, 0.1)
    out = ops.sparse_mla_attention(q.to(DEV), cache.to(DEV), idx.to(DEV), 0.1)
    _close(out, ref, 2e-2, 3e-2, f"sparse mla topk={topk}")


def test_bmm_heads():
    g = torch.Generator().manual_seed(1)
    for T, N, K, D in [(16, 16, 128, 512), (7, 128, 512, 128), (300, 4, 128, 512)]:
        x = (torch.randn(T, N, K, generator=g) * 0.5).bfloat16()
        w = (torch.randn(N, K, D, generator=g) * 0.05).bfloat16()
        ref = torch.einsum("tnk,nkd->tnd", x.float(), w.float())
        out = ops.bmm_heads(x.to(DEV), w.to(DEV))
        _close(out, ref, 0.03, 0.03, f"bmm_heads {T},{N},{K},{D}")


def test_deepseek_engine_gpu():
    cfg = tiny(deepseek_v3(fp8=False), num_layers=3, first_dense_layers=1, vocab_size=1024, hidden_size=512,
               num_heads=16, num_kv_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=1024,
               num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, n_group=4, topk_group=2,
               max_position=2048, rope_scaling=RopeScaling(type="yarn", factor=4.0, original_max_position=512,
                                                           mscale=1.0, mscale_all_dim=1.0), num_mtp_layers=0)
    outs = []
    for eager in (True, False):
        llm = LLM(cfg, device="cuda", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=32,
                  enforce_eager=eager, seed=2)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (90, 11)]
        outs.append([o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))])
    assert outs[0] == outs[1]


def test_indexer_logits_and_topk():
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.reference import basic as rb
    g = torch.Generator().manual_seed(4)
    bs, H = 64, 64
    spec = [(1, 700), (2, 131), (1, 3000), (40, 40)]  # (q_len, seq_len): decode rows, spec rows, a prefill
    B = len(spec)
    seq_lens = [s for _, s in spec]
    nblk = sum(-(-s // bs) for s in seq_lens) + 2
    bt = torch.zeros(B, max(-(-s // bs) for s in seq_lens) + 1, dtype=torch.int32)
    k = 1
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = torch.arange(k, k + n)
        k += n
    cache = torch.zeros(nblk + 1, bs, 132, dtype=torch.uint8)
    keys = torch.randn(sum(seq_lens), 128, generator=g)
    slots, off = [], 0
    for b, s in enumerate(seq_lens):
        pos = torch.arange(s)
        slots.append(bt[b, pos // bs].long() * bs + pos % bs)
    ra.indexer_k_quant_and_cache(keys, cache, torch.cat(slots))
    qsl = torch.tensor([0] + list(torch.tensor([q for q, _ in spec]).cumsum(0)), dtype=torch.int32)
    T = int(qsl[-1])
    q = torch.randn(T, H, 128, generator=g)
    qq, qs_ = rb.quant_fp8_per_group(q.reshape(T * H, 128), 128, True)
    qq, qs_ = qq.view(T, H, 128), qs_.view(T, H)
    w = torch.randn(T, H, generator=g) * 0.1
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    topk = 256
    want = ops.indexer_topk(qq, qs_, w, cache, bt, sl, qsl, topk)
    got = ops.indexer_topk(qq.to(DEV), qs_.to(DEV), w.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), qsl.to(DEV), topk)
    got = got.cpu()
    # same number of selected keys per row, and (up to ties / rounding at the cut) the same sets
    for t in range(T):
        a, b = set(want[t][want[t] >= 0].tolist()), set(got[t][got[t] >= 0].tolist())
        assert len(a) == len(b), (t, len(a), len(b))
        assert len(a & b) >= 0.97 * len(a), (t, len(a & b), len(a))
    # top-k kernel alone against torch.topk
    x = torch.randn(5, 5000, device=DEV)
    x[2, 100:200] = 1.5  # ties at the cut
    out = torch.empty(5, 512, dtype=torch.int32, device=DEV)
    lens = torch.tensor([5000, 300, 5000, 4097, 512], dtype=torch.int32, device=DEV)
    _ext.C().topk_rows(out, x, lens)
    for r in range(5):
        n = int(lens[r])
        sel = out[r][out[r] >= 0].long()
        kk = min(512, n)
        assert sel.numel() == kk and len(set(sel.tolist())) == kk and int(sel.max()) < n
        ref_vals = x[r, :n].topk(kk).values.sort().values
        assert torch.equal(x[r, sel].sort().values, ref_vals)


@pytest.mark.parametrize("fp8", [False, True])
def test_deepseek_mtp_speculative_engine_gpu(fp8):
    """MLA + MoE target with one MTP draft layer and one speculative token: verification keeps the target's greedy
    tokens, whatever the (random-init) draft proposes; q_len = 2 rows run through the decode attention path."""
    cfg = tiny(deepseek_v3(fp8=fp8), num_layers=3, first_dense_layers=1, vocab_size=1024, hidden_size=512,
               num_heads=16, num_kv_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=1024,
               num_experts=16, num_experts_per_tok=16, moe_intermediate_size=256, n_group=1, topk_group=1,
               max_position=2048, rope_scaling=RopeScaling(type="yarn", factor=4.0, original_max_position=512,
                                                           mscale=1.0, mscale_all_dim=1.0), num_mtp_layers=1)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (90, 11, 40)]
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    kw = dict(device="cuda", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=32, seed=2)
    base = [o.token_ids for o in LLM(cfg, enforce_eager=True, **kw).generate(prompts, sp)]
    for eager in (True, False):
        llm = LLM(cfg, enforce_eager=eager, speculative_config={"method": "mtp", "num_speculative_tokens": 1}, **kw)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        st = llm.engine.stats
        assert st["spec_proposed"] > 0
        flat_a, flat_b = sum(got, []), sum(base, [])
        # q_len = 2 verification rows and q_len = 1 rows take different kernel shapes (bf16): allow rare flips
        assert sum(x == y for x, y in zip(flat_a, flat_b)) >= 0.85 * len(flat_b), (eager, got, base)


def test_indexer_prep_fused_matches_unfused_ops():
    """One-launch indexer preparation (K LayerNorm, rotary on q / k, e4m3 + power-of-two scales, key-cache write,
    head weight x q scale) against the same steps as separate ops."""
    from vllm_kunlun_b200.models.layers import get_cos_sin_cache
    from vllm_kunlun_b200.config import RopeScaling
    from vllm_kunlun_b200.ops import _ext
    T, H, bs, nblk = 37, 64, 64, 6
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.randn(T, H, 128, device=DEV, generator=g).bfloat16()
    k = (torch.randn(T, 128, device=DEV, generator=g) * 2 + 0.3).bfloat16()
    lw = (torch.rand(128, device=DEV, generator=g) + 0.5).bfloat16()
    lb = (torch.randn(128, device=DEV, generator=g) * 0.1).bfloat16()
    hw = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    pos = torch.randint(0, 4000, (T,), device=DEV, generator=g)
    slots = torch.randperm(nblk * bs, device=DEV, generator=g)[:T].long()
    slots[3] = -1  # a padded token writes nothing
    cos_sin = get_cos_sin_cache(64, 4096, 10000.0, RopeScaling(), DEV)
    cache = torch.zeros(nblk, bs, 132, dtype=torch.uint8, device=DEV)
    q8, w = _ext.C().indexer_prep(q, k, lw, lb, pos, cos_sin, hw, 0.0125, cache, slots, 1e-6, True, 0)
    # the same steps, unfused
    kn = torch.nn.functional.layer_norm(k.float(), (128,), lw.float(), lb.float(), 1e-6).bfloat16()
    q_pe, k_pe = ops.rope(q[..., :64].reshape(T, -1).contiguous(), kn[:, :64].contiguous(), pos, cos_sin, 64, True)
    q2 = torch.cat([q_pe.view(T, H, 64), q[..., 64:]], -1)
    k2 = torch.cat([k_pe.view(T, 64), kn[:, 64:]], -1)
    cache2 = torch.zeros_like(cache)
    ops.indexer_k_quant_and_cache(k2.contiguous(), cache2, slots, True)
    q8r, qs = ops.quant_fp8_per_group(q2.reshape(T * H, 128).contiguous(), 128, True)
    torch.cuda.synchronize()
    wr = hw.float() * 0.0125 * qs.view(T, H).float()
    # scales are powers of two: identical unless an absolute maximum sits on a rounding edge of the LayerNorm
    deq = q8.view(torch.float8_e4m3fn).float() * (w / (hw.float() * 0.0125)).unsqueeze(-1)
    deq_r = q8r.view(T, H, 128).view(torch.float8_e4m3fn).float() * qs.view(T, H, 1).float()
    _close(deq, deq_r, 1e-6, 1e-6, "indexer q")
    _close(w, wr, 1e-7, 1e-6, "indexer head weights")
    (kq, ks), (kq_r, ks_r) = ra.indexer_cache_views(cache), ra.indexer_cache_views(cache2)
    kd = kq.contiguous().view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
    kd_r = kq_r.contiguous().view(torch.float8_e4m3fn).float() * ks_r.unsqueeze(-1)
    # LayerNorm statistics are summed in another order: a bf16 rounding may flip, which moves one e4m3 code
    _close(kd, kd_r, 0.07, 0.07, "indexer k rows")
    assert (kd != kd_r).float().mean() < 0.02


@pytest.mark.parametrize("t_lo_frac", [0.0, 0.37])
def test_indexer_logits_umma_matches_mma_sync_kernel(t_lo_frac):
    """tcgen05 indexer logits (keys on the UMMA M side, 4 tokens x 64 heads on the N side) against the mma.sync
    kernel on every visible key: prefill chunks with and without cached context, a decode row, requests that end
    inside a page, and a slice of the batch's tokens (as one tensor-parallel rank scores it)."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    from vllm_kunlun_b200.ops.mla_cuda import indexer_row_len
    from vllm_kunlun_b200.ops.reference import basic as rb
    g = torch.Generator().manual_seed(9)
    bs, H = 64, 64
    spec = [(300, 300), (1, 700), (77, 1100), (130, 130), (17, 64)]   # (q_len, seq_len)
    B = len(spec)
    seq_lens = [s for _, s in spec]
    nblk = sum(-(-s // bs) for s in seq_lens) + 2
    bt = torch.zeros(B, max(-(-s // bs) for s in seq_lens) + 1, dtype=torch.int32)
    k = 1
    for b, s in enumerate(seq_lens):
        n = -(-s // bs)
        bt[b, :n] = torch.arange(k, k + n)
        k += n
    cache = torch.zeros(nblk + 1, bs, 132, dtype=torch.uint8)
    keys = torch.randn(sum(seq_lens), 128, generator=g)
    slots = []
    for b, s in enumerate(seq_lens):
        pos = torch.arange(s)
        slots.append(bt[b, pos // bs].long() * bs + pos % bs)
    ra.indexer_k_quant_and_cache(keys, cache, torch.cat(slots))
    qsl = torch.tensor([0] + list(torch.tensor([q for q, _ in spec]).cumsum(0)), dtype=torch.int32)
    T = int(qsl[-1])
    q = torch.randn(T, H, 128, generator=g)
    qq, qs_ = rb.quant_fp8_per_group(q.reshape(T * H, 128), 128, True)
    w = (torch.randn(T, H, generator=g) * 0.1 * qs_.view(T, H)).contiguous()
    req = torch.repeat_interleave(torch.arange(B, dtype=torch.int32), (qsl[1:] - qsl[:-1]).long())
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    C = _ext.C()
    d = lambda x: x.to(DEV)
    lo = int(T * t_lo_frac)
    hi = T if t_lo_frac == 0.0 else T - 5
    ld = 1536
    qd = d(qq.view(T, H, 128).view(torch.uint8))[lo:hi].contiguous()
    wd = d(w)[lo:hi].contiguous()
    a = torch.full((hi - lo, ld), float("nan"), device=DEV)
    b_ = torch.full((hi - lo, ld), float("nan"), device=DEV)
    C.indexer_logits(a, qd, wd, d(cache), d(bt), d(sl), d(qsl), d(req)[lo:hi].contiguous(), lo)
    C.indexer_logits_umma(b_, qd, wd, d(cache), d(bt), d(sl), d(qsl), max(q for q, _ in spec), lo)
    torch.cuda.synchronize()
    check_status()
    rl = indexer_row_len(d(sl), d(qsl), d(req), T)[lo:hi].cpu()
    a, b_ = a.cpu(), b_.cpu()
    for t in range(hi - lo):
        n = int(rl[t])
        assert torch.isfinite(b_[t, :n]).all(), (t, n)
        # exact e4m3 products, fp32 sums in another order
        torch.testing.assert_close(b_[t, :n], a[t, :n], atol=2e-4, rtol=2e-4)
        up = min(ld, -(-n // 128) * 128)
        assert (b_[t, n:up] == float("-inf")).all(), (t, n)


def test_gather_mla_rows_bf16_and_fp8():
    """Row gather out of the paged latent cache, plain and with the 656-byte fp8 rows de-quantised on the way."""
    from vllm_kunlun_b200.ops import _ext
    g = torch.Generator(device=DEV).manual_seed(2)
    nblk, bs, T = 7, 64, 150
    kvc = torch.randn(T, 512, device=DEV, generator=g).bfloat16()
    kpe = torch.randn(T, 64, device=DEV, generator=g).bfloat16()
    slots = torch.randperm(nblk * bs, device=DEV, generator=g)[:T].long()
    c16 = torch.zeros(nblk, bs, 576, device=DEV, dtype=torch.bfloat16)
    c8 = torch.zeros(nblk, bs, 656, device=DEV, dtype=torch.uint8)
    ops.concat_and_cache_mla(kvc, kpe, c16, slots)
    ops.concat_and_cache_mla(kvc, kpe, c8, slots)
    pick = torch.cat([slots[:100].int(), torch.tensor([-1, nblk * bs + 5], device=DEV, dtype=torch.int32)])
    o16 = torch.full((pick.numel(), 576), float("nan"), device=DEV, dtype=torch.bfloat16)
    o8 = torch.full_like(o16, float("nan"))
    _ext.C().gather_mla_rows(o16, c16, pick)
    _ext.C().gather_mla_rows(o8, c8, pick)
    torch.cuda.synchronize()
    want = torch.cat([kvc, kpe], -1)[:100]
    assert torch.equal(o16[:100], want) and (o16[100:] == 0).all() and (o8[100:] == 0).all()
    ref8 = ra.dequant_mla_fp8_rows(c8.cpu().view(-1, 656)[pick[:100].long().cpu()]).bfloat16()
    assert torch.equal(o8[:100].cpu(), ref8)
    _close(o8[:100], want.float().cpu(), 0.15, 0.08, "fp8_ds_mla rows")


def test_deepseek_sparse_engine_fp8_latent_cache():
    """V3.2-shaped tiny model with ``kv_cache_dtype='fp8_ds_mla'``: the attention reads the quantised cache through
    the gather + de-quantise path; greedy tokens mostly agree with the 16-bit cache (the cache is lossy)."""
    from vllm_kunlun_b200.config import deepseek_v3
    cfg = tiny(deepseek_v3(fp8=False, sparse=True), num_layers=2, first_dense_layers=1, vocab_size=512, hidden_size=512,
               num_heads=16, num_kv_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=1024,
               num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, n_group=1, topk_group=1,
               max_position=2048, num_mtp_layers=0, index_topk=64)
    prompts = [torch.randint(0, 512, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (200, 70)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    toks = {}
    for kvd in ("auto", "fp8_ds_mla"):
        llm = LLM(cfg, device="cuda", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=24, seed=1,
                  kv_cache_dtype=kvd)
        caches = llm.engine.runner.kv_caches
        first = caches[min(caches)]
        assert (first[0].dtype == torch.uint8) == (kvd == "fp8_ds_mla")
        toks[kvd] = [o.token_ids for o in llm.generate(prompts, sp)]
        torch.cuda.synchronize()
    assert all(len(t) == 6 for t in toks["fp8_ds_mla"])
    same = sum(a == b for x, y in zip(toks["auto"], toks["fp8_ds_mla"]) for a, b in zip(x, y))
    assert same >= 6, toks   # at least half of the 12 greedy tokens


@pytest.mark.parametrize("N", [16, 3])
@pytest.mark.parametrize("causal", [True, False])
def test_mla_prefill_umma_kernel(N, causal):
    """MLA prefill in the up-projected form on tcgen05 (192-dim q / k from three 64-dim blocks, the rotary block
    shared by the heads; 128-dim v; contiguous keys per request) vs the fp32 oracle: key counts on and off the
    128-key tile edge, query tiles that end inside a tile, a request without keys (not causal), a strided view as
    the rotary-key tensor, and the log-sum-exp output."""
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    g = torch.Generator().manual_seed(N + 7 * causal)
    if causal:
        q_lens = [1, 64, 127, 128, 129, 300, 517]
        kv_lens = list(q_lens)
    else:
        q_lens = [5, 130, 64, 256, 77]
        kv_lens = [700, 128, 0, 129, 1]
    T, R = sum(q_lens), sum(kv_lens)
    q = (torch.randn(T, N, 192, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(R, N * 256, generator=g) * 0.5).bfloat16()
    rows = (torch.randn(R, 576, generator=g) * 0.5).bfloat16()      # k_pe = the last 64 columns of gathered rows
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    ks = torch.tensor([0] + list(torch.tensor(kv_lens).cumsum(0))[:-1], dtype=torch.int32)
    kl = torch.tensor(kv_lens, dtype=torch.int32)
    scale = 192 ** -0.5
    want, want_lse = ra.mla_prefill(q, kv, rows[:, 512:], ks, kl, qsl, causal, scale)
    rows_d = rows.to(DEV)
    out, lse = ops.mla_prefill_attention(q.to(DEV), kv.to(DEV), rows_d[:, 512:], ks.to(DEV), kl.to(DEV), qsl.to(DEV),
                                         causal, scale, max(q_lens))
    check_status()
    _close(out, want, 0.02, 0.03, f"mla prefill out N={N} causal={causal}")
    fin = torch.isfinite(want_lse)
    assert bool((torch.isfinite(lse.cpu()) == fin).all())
    _close(lse.cpu()[fin], want_lse[fin], 0.02, 0.01, "mla prefill lse")
    if not causal:      # the request without keys: untouched rows (zeros / -inf as preset)
        s, e = int(qsl[2]), int(qsl[3])
        assert float(out[s:e].abs().max()) == 0.0 and bool(torch.isinf(lse[s:e]).all())


def test_mla_attention_prefill_form_matches_absorbed_form_gpu():
    """One MLA layer on the GPU: a 200-token prompt under a 140-token step budget (the second step has 60 new tokens
    over 140 cached ones, read through three passes of a 64-token context workspace, and a 7-token request beside
    it that stays on the absorbed form); the up-projected form must give the rows of the absorbed form."""
    from vllm_kunlun_b200.attention.metadata import ForwardContext, set_forward_context
    from vllm_kunlun_b200.models.deepseek import MLAAttention
    cfg = tiny(deepseek_v3(fp8=False), num_layers=2, first_dense_layers=1, vocab_size=1024, hidden_size=512,
               num_heads=16, num_kv_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
               qk_rope_head_dim=64, v_head_dim=128, head_dim=192, rotary_dim=64, intermediate_size=1024,
               num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, n_group=4, topk_group=2,
               max_position=2048, rope_scaling=RopeScaling(type="yarn", factor=4.0, original_max_position=512,
                                                           mscale=1.0, mscale_all_dim=1.0), num_mtp_layers=0)
    llm = LLM(cfg, device="cuda", block_size=64, max_model_len=512, max_num_seqs=4, num_gpu_blocks=32,
              max_num_batched_tokens=140, enforce_eager=True, seed=3)
    eng = llm.engine
    attn = eng.runner.model.layers["0"].self_attn
    eng.add_request(list(range(200)), SamplingParams(max_tokens=1))
    eng.add_request(list(range(7)), SamplingParams(max_tokens=1))
    g = torch.Generator().manual_seed(5)
    old = (MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_CTX_BYTES, MLAAttention.PREFILL_MIN_QUERY)
    MLAAttention.PREFILL_MIN_QUERY = 16
    seen_chunks, mixed = [], []
    try:
        for step in range(2):
            sched = eng.scheduler.schedule()
            md, ids, _ = eng.runner.prepare(sched)
            hidden = (torch.randn(md.num_tokens, cfg.hidden_size, generator=g) * 0.5).bfloat16().to(DEV)
            with torch.inference_mode(), set_forward_context(ForwardContext(md, eng.runner.kv_caches, eng.pstate)):
                MLAAttention.PREFILL_FORM = False
                want = attn(hidden)
                md.extras.pop("mla_prefill_plan", None)
                MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_CTX_BYTES = True, 16 * 256 * 2 * 64
                got = attn(hidden)
                plan = md.extras["mla_prefill_plan"]
            assert plan is not None
            seen_chunks.append(len(plan["chunks"]))
            mixed.append(plan["rest"] is not None)
            _close(got, want, 0.03, 0.05, f"step {step}")
            for sr in sched.scheduled:
                sr.req.num_computed_tokens += sr.num_new_tokens
    finally:
        MLAAttention.PREFILL_FORM, MLAAttention.PREFILL_CTX_BYTES, MLAAttention.PREFILL_MIN_QUERY = old
    assert seen_chunks == [0, 3] and mixed == [False, True], (seen_chunks, mixed)
