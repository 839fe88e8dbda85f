"""Schema inference and dispatcher registration of plain functions."""
from typing import List, Optional, Sequence, Tuple

import pytest
import torch

from vllm_kunlun_b200.schema import direct_register_custom_op, infer_schema


def test_infer_schema_spellings():
    def f(out: torch.Tensor, x: torch.Tensor, shape: Optional[List[int]] = None, eps: float = 1e-6) -> None: ...
    assert infer_schema(f, ["out"]) == "(Tensor(a!) out, Tensor x, SymInt[]? shape=None, float eps=1e-06) -> ()"

    def g(x: torch.Tensor, dims: list[int], w: torch.Tensor | None = None, *, neox: bool = True,
          mode: str = "a") -> torch.Tensor: ...
    assert infer_schema(g) == '(Tensor x, SymInt[] dims, Tensor? w=None, *, bool neox=True, str mode="a") -> Tensor'

    def h(a: torch.Tensor, b: torch.Tensor, xs: Sequence[torch.Tensor], k: int = 2) -> Tuple[torch.Tensor, torch.Tensor]: ...
    assert infer_schema(h, ["a", "b"]) == "(Tensor(a!) a, Tensor(b!) b, Tensor[] xs, SymInt k=2) -> (Tensor, Tensor)"

    def many(x: torch.Tensor) -> tuple[torch.Tensor, ...]: ...
    assert infer_schema(many) == "(Tensor x) -> Tensor[]"


def test_infer_schema_rejects():
    def no_ann(x, y: int): ...
    def nested(x: List[List[int]]): ...
    def union(x: int | float): ...
    def var(*xs: int): ...
    def mut(n: int): ...
    for fn, kw in ((no_ann, {}), (nested, {}), (union, {}), (var, {}), (mut, {"mutates_args": ["n"]})):
        with pytest.raises(TypeError):
            infer_schema(fn, **kw)
    with pytest.raises(ValueError):
        infer_schema(mut, ["missing"])


def test_register_and_call():
    def scaled_add_(out: torch.Tensor, x: torch.Tensor, alpha: float = 1.0, idx: Optional[List[int]] = None) -> None:
        out.add_(x if idx is None else x[idx], alpha=alpha)

    def pair(x: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return x * k, x + k

    op = direct_register_custom_op("scaled_add_", scaled_add_, ["out"], namespace="b200_schema_test")
    out, x = torch.zeros(3), torch.arange(3.0)
    op(out, x, 2.0)
    torch.ops.b200_schema_test.scaled_add_(out, x, idx=[2, 2, 2])
    assert out.tolist() == [2.0, 4.0, 6.0]

    op2 = direct_register_custom_op("pair", pair, namespace="b200_schema_test",
                                    fake_impl=lambda x, k: (torch.empty_like(x), torch.empty_like(x)))
    a, b = op2(x, 3)
    assert a.tolist() == [0.0, 3.0, 6.0] and b.tolist() == [3.0, 4.0, 5.0]
    # the fake implementation lets a tracer run the op on meta tensors
    fa, fb = op2(torch.empty(5, device="meta"), 3)
    assert fa.shape == (5,) and fb.device.type == "meta"


def test_b200_namespace_ops_match_oracles():
    from vllm_kunlun_b200.ops.custom_ops import register_custom_ops
    from vllm_kunlun_b200.ops.reference import basic as rb

    register_custom_ops()
    register_custom_ops()  # idempotent
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(5, 64, generator=g), torch.randn(64, generator=g)
    assert torch.allclose(torch.ops.b200.rms_norm(x, w, 1e-6), rb.rmsnorm(x, w, 1e-6, False))
    res = torch.randn(5, 64, generator=g)
    want_out, want_res = rb.add_rmsnorm(x.clone(), res.clone(), w, 1e-6, False)
    x2, res2 = x.clone(), res.clone()
    assert torch.ops.b200.fused_add_rms_norm_(x2, res2, w, 1e-6) is None
    assert torch.allclose(x2, want_out) and torch.allclose(res2, want_res)
    h = torch.randn(5, 128, generator=g)
    assert torch.allclose(torch.ops.b200.act_and_mul(h), torch.nn.functional.silu(h[:, :64]) * h[:, 64:])
    wt = torch.randn(32, 64, generator=g)
    assert torch.allclose(torch.ops.b200.linear(x, wt), x @ wt.T, atol=1e-5)
    tw, ids = torch.ops.b200.moe_route(torch.randn(5, 8, generator=g), 2)
    assert tw.shape == (5, 2) and ids.shape == (5, 2)
    # fake implementations: shapes on meta tensors
    m = torch.empty(7, 128, device="meta")
    assert torch.ops.b200.act_and_mul(m).shape == (7, 64)
    assert torch.ops.b200.linear(torch.empty(7, 64, device="meta"), torch.empty(32, 64, device="meta")).shape == (7, 32)
    assert "Tensor(a!) x, Tensor(b!) residual" in str(torch.ops.b200.fused_add_rms_norm_.default._schema)


def test_every_dispatcher_op_has_a_schema_declared_mutations_and_a_fake_impl():
    """All ops of the table are defined, ops that write an argument say so in their schema, and a sample of them
    runs through the dispatcher on CPU tensors (oracle path) and on meta tensors (fake implementations)."""
    from vllm_kunlun_b200 import ops
    from vllm_kunlun_b200.ops.custom_ops import OPS, register_custom_ops
    register_custom_ops()
    assert len(OPS) >= 30
    for name, (fn, mutates, fake) in OPS.items():
        op = getattr(torch.ops.b200, name)
        schema = str(op.default._schema)
        assert name.endswith("_") == bool(mutates), name
        for arg in mutates:
            assert f"!) {arg}" in schema, (name, schema)   # Tensor(a!) arg
        if not mutates:
            assert "!" not in schema, (name, schema)
    g = torch.Generator().manual_seed(1)
    # rope, in place
    from vllm_kunlun_b200.ops.reference.basic import build_cos_sin_cache
    cs = build_cos_sin_cache(16, 64, 1e4, None)
    q, k = torch.randn(3, 2 * 16, generator=g), torch.randn(3, 16, generator=g)
    pos = torch.tensor([0, 5, 9])
    wq, wk = ops.rope(q.clone(), k.clone(), pos, cs, 16, True)
    q2, k2 = q.clone(), k.clone()
    torch.ops.b200.rotary_embedding_(q2, k2, pos, cs, 16, True)
    assert torch.allclose(q2, wq) and torch.allclose(k2, wk)
    # MLA cache write + attention through the dispatcher
    cache = torch.zeros(3, 64, 576)
    kv_c, k_pe = torch.randn(10, 512, generator=g), torch.randn(10, 64, generator=g)
    torch.ops.b200.concat_and_cache_mla_(kv_c, k_pe, cache, torch.arange(64, 74))
    assert torch.allclose(cache[1, :10, :512], kv_c) and torch.allclose(cache[1, :10, 512:], k_pe)
    qm = torch.randn(10, 2, 576, generator=g) * 0.1
    bt = torch.tensor([[1, 0]], dtype=torch.int32)
    out = torch.ops.b200.mla_attention(qm, cache, bt, torch.tensor([10], dtype=torch.int32),
                                       torch.tensor([0, 10], dtype=torch.int32), 0.1, 512, 10, 10)
    assert out.shape == (10, 2, 512)
    # routing variants and the fused MoE
    logits = torch.randn(6, 8, generator=g)
    w, ids = torch.ops.b200.moe_route(logits, 2, "sigmoid", True, torch.zeros(8), 4, 2, 2.5)
    assert w.shape == (6, 2) and int(ids.max()) < 8
    x = torch.randn(6, 32, generator=g)
    w13, w2 = torch.randn(8, 64, 32, generator=g) * 0.1, torch.randn(8, 32, 32, generator=g) * 0.1
    y = torch.ops.b200.fused_moe(x, w13, w2, w, ids)
    assert torch.allclose(y, ops.fused_moe(x, w13, w2, w, ids), atol=1e-5)
    # quantisers / quantised linears
    qx, sx = torch.ops.b200.quant_fp8_per_group(torch.randn(4, 256, generator=g))
    assert qx.dtype == torch.float8_e4m3fn and sx.shape == (4, 2)
    # sampling
    lg = torch.randn(4, 50, generator=g)
    assert torch.equal(torch.ops.b200.argmax(lg), lg.argmax(-1))
    lg2 = lg.clone()
    torch.ops.b200.apply_repetition_penalties_(lg2, torch.tensor([[1, 2], [3, 3], [0, 0], [7, 8]]),
                                               torch.tensor([2, 2, 0, 1], dtype=torch.int32), torch.full((4,), 2.0))
    assert not torch.equal(lg2, lg) and torch.equal(lg2[2], lg[2])
    # LoRA
    a = torch.randn(2, 4, 32, generator=g)
    b = torch.randn(2, 16, 4, generator=g)
    ids2 = torch.tensor([0, -1, 1, 0, 1, 1], dtype=torch.int32)
    h = torch.ops.b200.lora_shrink(x, a, ids2, 0.5)
    yo = torch.zeros(6, 16)
    torch.ops.b200.lora_expand_(h, b, ids2, yo, 0, True)
    assert yo[1].abs().sum() == 0 and yo[0].abs().sum() > 0
    # fake implementations on meta tensors give the shapes the real ops give
    M = lambda *s, dtype=torch.float32: torch.empty(*s, device="meta", dtype=dtype)  # noqa: E731
    assert torch.ops.b200.mla_attention(M(10, 2, 576), M(3, 64, 576), M(1, 2, dtype=torch.int32), M(1, dtype=torch.int32),
                                        M(2, dtype=torch.int32), 0.1, 512, 10, 10).shape == (10, 2, 512)
    fw, fi = torch.ops.b200.moe_route(M(6, 8), 2)
    assert fw.shape == (6, 2) and fi.dtype == torch.int32
    fq, fs = torch.ops.b200.quant_fp8_per_group(M(4, 256))
    assert fq.dtype == torch.float8_e4m3fn and fs.shape == (4, 2)
    assert torch.ops.b200.lora_shrink(M(6, 32), M(2, 4, 32), M(6, dtype=torch.int32)).shape == (6, 4)
    assert torch.ops.b200.indexer_topk(M(5, 64, 128), M(5, 64), M(5, 64), M(4, 64, 132, dtype=torch.uint8),
                                       M(1, 4, dtype=torch.int32), M(1, dtype=torch.int32), M(2, dtype=torch.int32),
                                       2048).shape == (5, 2048)
    assert torch.ops.b200.fused_add_rms_norm_(M(3, 8), M(3, 8), M(8), 1e-6) is None
