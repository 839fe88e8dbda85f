"""Dispatcher ops (``torch.ops.b200.*``) over the kernels, for hosts that trace models instead of calling Python.

The engine of this package calls ``ops.*`` directly.  A host that captures graphs by tracing (vLLM's compiled
mode, ``torch.export``) needs ops that the dispatcher knows: a schema, declared mutations, and a fake
implementation for shape propagation.  The reference wraps its vendor kernels the same way
(``vllm_kunlun/ops/_custom_ops.py``: ``_C::rmsnorm`` :303-340, ``_C::add_rmsnorm`` :255-300,
``_C::silu_and_mul`` :699-716, ``_C::rotary_embedding`` :993-1028).  Dispatcher ops may not return an alias of an
argument, so the in-place kernels are exposed in mutating form (trailing underscore, ``-> ()``), the others in
functional form."""
from typing import Optional, Tuple

import torch

from .. import ops
from ..schema import direct_register_custom_op

_done = False


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool = False) -> torch.Tensor:
    return ops.rmsnorm(x, weight, eps, gemma)


def fused_add_rms_norm_(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                        gemma: bool = False) -> None:
    """``residual += x; x = norm(residual) * weight``, both in place."""
    out, res = ops.add_rmsnorm(x, residual, weight, eps, gemma)
    if out.data_ptr() != x.data_ptr():  # the CPU oracle returns new tensors
        x.copy_(out)
        residual.copy_(res)


def act_and_mul(x: torch.Tensor, act: str = "silu") -> torch.Tensor:
    return ops.act_and_mul(x, act)


def rotary_embedding_(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
                      head_dim: int, neox: bool = True) -> None:
    q2, k2 = ops.rope(q, k, positions, cos_sin_cache, head_dim, neox)
    if q2.data_ptr() != q.data_ptr():
        q.copy_(q2)
        k.copy_(k2)


def reshape_and_cache_(k: torch.Tensor, v: torch.Tensor, kv_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    ops.reshape_and_cache(k, v, kv_cache, slot_mapping)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return ops.linear(x, weight, bias)


def moe_route(logits: torch.Tensor, k: int, scoring: str = "softmax",
              renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    w, ids = ops.moe_route(logits, k, scoring, renormalize)[:2]
    return w, ids


def _fake_half(x, act="silu"):
    return x.new_empty(*x.shape[:-1], x.shape[-1] // 2)


def _fake_linear(x, weight, bias=None):
    return x.new_empty(*x.shape[:-1], weight.shape[0])


def _fake_route(logits, k, scoring="softmax", renormalize=True):
    return (logits.new_empty(logits.shape[0], k, dtype=torch.float32),
            logits.new_empty(logits.shape[0], k, dtype=torch.int32))


def register_custom_ops() -> None:
    """Define the ``b200`` namespace once per process (``vllm.general_plugins`` entry point ``b200_ops``)."""
    global _done
    if _done:
        return
    _done = True
    direct_register_custom_op("rms_norm", rms_norm, fake_impl=lambda x, weight, eps, gemma=False: torch.empty_like(x))
    direct_register_custom_op("fused_add_rms_norm_", fused_add_rms_norm_, ["x", "residual"],
                              fake_impl=lambda x, residual, weight, eps, gemma=False: None)
    direct_register_custom_op("act_and_mul", act_and_mul, fake_impl=_fake_half)
    direct_register_custom_op("rotary_embedding_", rotary_embedding_, ["q", "k"],
                              fake_impl=lambda q, k, positions, cos_sin_cache, head_dim, neox=True: None)
    direct_register_custom_op("reshape_and_cache_", reshape_and_cache_, ["kv_cache"],
                              fake_impl=lambda k, v, kv_cache, slot_mapping: None)
    direct_register_custom_op("linear", linear, fake_impl=_fake_linear)
    direct_register_custom_op("moe_route", moe_route, fake_impl=_fake_route)
