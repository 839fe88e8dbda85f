"""MoE / fp8 CUDA kernels vs the fp32 oracles (B200)."""
import pytest
import torch

from vllm_kunlun_b200 import LLM, SamplingParams, ops
from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
from vllm_kunlun_b200.ops.reference import basic as rb
from vllm_kunlun_b200.ops.reference import moe as rm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, name=""):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    bad = (err > atol + rtol * b.abs()).float().mean().item()
    assert bad < 2e-3, f"{name}: {bad:.4%} elements off, max err {err.max().item():.4g}"


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (16, 128, 8), (77, 256, 8), (5, 32, 4), (300, 64, 6)])
def test_route_softmax(T, E, k):
    # bf16 logits tie often; ties may resolve to different experts with equal weight, so compare
    # the sorted weights and check that every returned weight belongs to its returned expert
    lg = torch.randn(T, E, device=DEV).bfloat16()
    p = lg.float().softmax(-1).cpu()
    for renorm in (True, False):
        w, ids = ops.moe_route(lg, k, "softmax", renorm)
        rw, rids = rm.route_softmax_topk(lg.cpu(), k, renorm)
        _close(w.sort(-1).values, rw.sort(-1).values, 1e-4, 1e-3, "softmax weights")
        own = p.gather(1, ids.cpu().long())
        if renorm:
            own = own / own.sum(-1, keepdim=True)
        _close(w, own, 1e-4, 1e-3, "weight/expert pairing")
        assert all(len(set(r)) == k for r in ids.cpu().tolist())
    lg32 = torch.randn(T, E, device=DEV)
    w, ids = ops.moe_route(lg32, k, "softmax", True)
    rw, rids = rm.route_softmax_topk(lg32.cpu(), k, True)
    assert torch.equal(ids.cpu().sort(-1).values, rids.sort(-1).values)
    w, ids = ops.moe_route(lg32, k, "softmax_after_topk")
    rw, rids = rm.route_topk_then_softmax(lg32.cpu(), k)
    assert torch.equal(ids.cpu().sort(-1).values, rids.sort(-1).values)
    _close(w.sort(-1).values, rw.sort(-1).values, 1e-4, 1e-3, "topk-softmax weights")


@pytest.mark.parametrize("T", [1, 16, 130])
def test_route_sigmoid_group(T):
    E, k = 256, 8
    lg = torch.randn(T, E, device=DEV)
    bias = (torch.randn(E, device=DEV) * 0.1)
    w, ids = ops.moe_route(lg, k, "sigmoid", True, bias, 8, 4, 2.5)
    rw, rids = rm.route_sigmoid_group_topk(lg.cpu(), bias.cpu(), k, 8, 4, True, 2.5)
    assert torch.equal(ids.cpu().sort(-1).values, rids.sort(-1).values)
    _close(w.sort(-1).values, rw.sort(-1).values, 1e-4, 1e-3, "sigmoid weights")


@pytest.mark.parametrize("T,N,K", [(16, 512, 1024), (1, 256, 128), (100, 1536, 2048), (300, 384, 7168)])
def test_fp8_linear(T, N, K):
    g = torch.Generator().manual_seed(T + N)
    w = torch.randn(N, K, generator=g) * 0.02
    q, s = rb.quant_fp8_block(w)
    x = torch.randn(T, K, generator=g)
    ref = ops.fp8_linear(x, q, s, out_dtype=torch.float32)
    out = ops.fp8_linear(x.to(DEV).bfloat16(), q.to(DEV), s.to(DEV))
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    torch.cuda.synchronize()
    check_status()
    _close(out, ref, 0.03 * (K / 1024) ** 0.5, 0.05, f"fp8 linear {T}x{N}x{K}")


def test_quant_fp8_group():
    x = torch.randn(37, 512, device=DEV).bfloat16()
    q, s = ops.quant_fp8_per_group(x)
    rq, rs = rb.quant_fp8_per_group(x.cpu())
    _close(s, rs, 1e-6, 1e-3, "scales")
    deq = q.float().reshape(37, 4, 128) * s.unsqueeze(-1)
    _close(deq.reshape(37, 512), x, 0.02, 0.07, "dequant")


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("T,E,k,H,I", [(16, 128, 8, 2048, 768), (1, 16, 2, 256, 128), (200, 32, 4, 512, 256)])
def test_fused_moe(fp8, T, E, k, H, I):
    g = torch.Generator().manual_seed(E + T)
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.03)
    w2 = (torch.randn(E, H, I, generator=g) * 0.03)
    tw, ids = rm.route_softmax_topk(torch.randn(T, E, generator=g), k)
    if fp8:
        q13, s13 = rb.quant_fp8_block(w13)
        q2, s2 = rb.quant_fp8_block(w2)
        ref = rm.fused_moe(x.float(), q13, q2, tw, ids, w13_scale=s13, w2_scale=s2)
        out = ops.fused_moe(x.to(DEV), q13.to(DEV), q2.to(DEV), tw.to(DEV), ids.to(DEV), w13_scale=s13.to(DEV),
                            w2_scale=s2.to(DEV))
        tol = 0.06
    else:
        w13b, w2b = w13.bfloat16(), w2.bfloat16()
        ref = rm.fused_moe(x.float(), w13b.float(), w2b.float(), tw, ids)
        out = ops.fused_moe(x.to(DEV), w13b.to(DEV), w2b.to(DEV), tw.to(DEV), ids.to(DEV))
        tol = 0.03
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    torch.cuda.synchronize()
    check_status()
    _close(out, ref, tol * ref.abs().max().item(), 0.05, f"fused_moe fp8={fp8}")


def test_fused_moe_expert_map():
    g = torch.Generator().manual_seed(3)
    T, E, k, H, I = 40, 16, 4, 256, 128
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.03).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) * 0.03).bfloat16()
    tw, ids = rm.route_softmax_topk(torch.randn(T, E, generator=g), k)
    full = rm.fused_moe(x.float(), w13.float(), w2.float(), tw, ids)
    acc = torch.zeros_like(full)
    for r in range(2):
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[r * 8:(r + 1) * 8] = torch.arange(8, dtype=torch.int32)
        acc += ops.fused_moe(x.to(DEV), w13[r * 8:(r + 1) * 8].to(DEV), w2[r * 8:(r + 1) * 8].to(DEV), tw.to(DEV),
                             ids.to(DEV), expert_map=emap.to(DEV)).float().cpu()
    _close(acc, full, 0.03 * full.abs().max().item(), 0.05, "expert-parallel halves")


@pytest.mark.parametrize("fp8", [False, True])
def test_moe_engine_gpu(fp8):
    cfg = tiny(qwen3_30b_a3b(fp8=fp8), num_layers=2, vocab_size=1024, hidden_size=512, num_heads=8, num_kv_heads=2,
               head_dim=64, intermediate_size=1024, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256,
               max_position=2048)
    outs = []
    for eager in (True, False):
        llm = LLM(cfg, device="cuda", block_size=16, max_model_len=256, max_num_seqs=4, num_gpu_blocks=64,
                  enforce_eager=eager, seed=11)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 7)]
        outs.append([o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))])
    assert outs[0] == outs[1]


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("T,k,E", [(1, 8, 128), (16, 8, 128), (128, 8, 64), (100, 4, 32)])
def test_small_batch_fusion_is_bitwise_equal(fp8, T, k, E):
    """One-launch permute (+ fp8 quantisation) and the fused activation + quantiser give the same bits as the
    separate kernels: rows are processed independently of where they sit in the permuted buffer."""
    from vllm_kunlun_b200.models.moe import _quant_block_device
    from vllm_kunlun_b200.ops import moe_cuda
    torch.manual_seed(T + k)
    H, I = 512, 256
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    w13 = torch.randn(E, 2 * I, H, device=DEV) * 0.05
    w2 = torch.randn(E, H, I, device=DEV) * 0.05
    s13 = s2 = None
    if fp8:
        q13, q2 = [_quant_block_device(w13[e]) for e in range(E)], [_quant_block_device(w2[e]) for e in range(E)]
        w13, s13 = torch.stack([a for a, _ in q13]), torch.stack([b for _, b in q13])
        w2, s2 = torch.stack([a for a, _ in q2]), torch.stack([b for _, b in q2])
    else:
        w13, w2 = w13.bfloat16(), w2.bfloat16()
    wts, ids = ops.moe_route(torch.randn(T, E, device=DEV), k, "softmax", True)
    emap = torch.arange(E, dtype=torch.int32, device=DEV)
    emap[E // 2:] = -1  # half of the experts live elsewhere
    outs = []
    for on in (True, False):
        moe_cuda.SMALL_BATCH_FUSION[0] = on
        outs.append(ops.fused_moe(x, w13[: E // 2].contiguous(), w2[: E // 2].contiguous(), wts, ids, "silu", None, None,
                                  None if s13 is None else s13[: E // 2].contiguous(),
                                  None if s2 is None else s2[: E // 2].contiguous(), (128, 128), emap))
    moe_cuda.SMALL_BATCH_FUSION[0] = True
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("T,E,K", [(1, 128, 2048), (16, 128, 2048), (64, 256, 7168), (5, 32, 512)])
def test_router_gemm_small(T, E, K):
    torch.manual_seed(T)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(E, K, device=DEV) * 0.05).bfloat16()
    b = torch.randn(E, device=DEV).bfloat16()
    got = ops.router_gemm(x, w, b)
    assert got.dtype == torch.float32
    want = x.float() @ w.float().T + b.float()
    torch.testing.assert_close(got, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("T,N,K,splits", [(16, 2048, 4096, 0), (1, 128, 128, 0), (7, 384, 1024, 2), (32, 520, 7168, 4),
                                          (16, 512, 1024, 8), (24, 256, 2048, 1), (3, 1536, 640, 0)])
def test_gemm_decode_fp8_cluster_splitk(T, N, K, splits):
    """fp8 block-scaled decode kernel (one TMEM buffer per 128-wide k-block, scales applied in the epilogue warps)
    against fp32 arithmetic on the SAME quantised operands."""
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    g = torch.Generator().manual_seed(T + N + K)
    w = torch.randn(N, K, generator=g) * 0.05
    q, s = rb.quant_fp8_block(w)
    x = torch.randn(T, K, generator=g).bfloat16()
    bias = torch.randn(N, generator=g).bfloat16()
    C = _ext.C()
    xq, st = C.quant_fp8_group(x.to(DEV), False, None, 4)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    C.gemm_decode_fp8(out, xq, q.to(DEV).view(torch.uint8), bias.to(DEV), st, s.to(DEV), splits)
    torch.cuda.synchronize()
    check_status()
    xd = xq.view(torch.float8_e4m3fn).float().cpu() * st[:, :T].T.cpu().repeat_interleave(128, 1)[:, :K]
    wd = q.float() * s.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    ref = xd @ wd.T + bias.float()
    # exact products, fp32 sums: what is left is the bf16 output rounding and the order of the K sum
    _close(out, ref, 2e-3 * (K / 64) ** 0.5, 6e-3, f"gemm_decode_fp8 {T}x{N}x{K}/{splits}")
    out2 = torch.empty_like(out)
    C.gemm_decode_fp8(out2, xq, q.to(DEV).view(torch.uint8), bias.to(DEV), st, s.to(DEV), splits)
    assert torch.equal(out, out2)


def test_fp8_projection_decode_batches_read_the_fp8_weight():
    """A quantised layer keeps ONE copy of its weight; 16-row and 300-row calls agree with the de-quantised oracle."""
    from vllm_kunlun_b200.models.layers import ReplicatedLinear
    from vllm_kunlun_b200.models.moe import _quant_block_device
    torch.manual_seed(0)
    lin = ReplicatedLinear(1024, 512, dtype=torch.bfloat16, device=DEV, quant="fp8")
    q, s = _quant_block_device(torch.randn(512, 1024, device=DEV) * 0.05)
    lin.weight.data.copy_(q)
    lin.weight_scale_inv.data.copy_(s)
    lin.method.process_weights_after_loading(lin)
    assert not hasattr(lin, "weight_16bit")
    x = torch.randn(300, 1024, device=DEV).bfloat16()
    big = lin(x)            # grouped block-scaled kernel
    small = lin(x[:16])     # cluster split-K decode kernel
    wd = q.float() * s.repeat_interleave(128, 0).repeat_interleave(128, 1)
    ref = x.float() @ wd.T
    _close(small, ref[:16], 0.25, 0.1, "fp8 decode path")  # activations are quantised to e4m3 per 128 columns
    _close(big, ref, 0.25, 0.1, "fp8 grouped path")
    _close(small, big[:16], 2e-2, 2e-2, "the two kernels compute the same quantised product")


@pytest.mark.parametrize("scoring,E,k,ng,tg", [("softmax", 128, 8, 1, 1), ("sigmoid", 256, 8, 8, 4), ("softmax_after_topk", 32, 4, 1, 1)])
def test_router_and_route_fused_equals_two_kernels(scoring, E, k, ng, tg):
    torch.manual_seed(E)
    T, K = 16, 2048
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(E, K, device=DEV) * 0.05).bfloat16()
    bias = torch.randn(E, device=DEV) * 0.1 if scoring == "sigmoid" else None
    from vllm_kunlun_b200.ops import _ext
    from vllm_kunlun_b200.ops.moe_cuda import _MODES
    w1, i1 = _ext.C().router_route_small(x, w, None, bias, k, _MODES[scoring], True, ng, tg, 2.5)  # the fused kernel itself
    w3, i3 = ops.router_and_route(x, w, None, k, scoring, True, bias, ng, tg, 2.5)               # dispatcher
    assert torch.equal(i3.sort(-1).values, i1.sort(-1).values)
    w2, i2 = ops.moe_route(ops.router_gemm(x, w, None), k, scoring, True, bias, ng, tg, 2.5)
    # both read fp32 logits produced by the same dot-product order
    assert torch.equal(i1.sort(-1).values, i2.sort(-1).values)
    torch.testing.assert_close(w1.sort(-1).values, w2.sort(-1).values, atol=1e-5, rtol=1e-5)
