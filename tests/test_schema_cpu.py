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
