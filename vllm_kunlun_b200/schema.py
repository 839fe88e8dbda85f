"""Operator schemas from Python signatures, and registration of plain functions as ``torch.ops.<ns>.<name>``.

The engine of this package calls its kernels as plain functions; a tracing host (vLLM's compiled graphs, or
``torch.export``) wants dispatcher ops with a schema and a fake (meta) implementation instead.  This module turns
an annotated function into such an op.  It plays the role of the reference's schema helper
(``vllm_kunlun/schema.py:1-117``, a re-implementation of ``direct_register_custom_op`` that accepts ``list[int]``
and PEP-604 optionals, which ``torch.library.infer_schema`` of older releases rejected), built here directly on
the type objects: every annotation is reduced to (base type, is-list, is-optional) and printed in the dispatcher's
grammar, so ``Optional[List[int]]``, ``list[int] | None`` and ``typing.Sequence[int]`` all print ``SymInt[]?``.
"""
import inspect
import types
import typing
from typing import Callable, Optional, Sequence

import torch

_BASE = {torch.Tensor: "Tensor", int: "SymInt", float: "float", bool: "bool", str: "str",
         torch.dtype: "ScalarType", torch.device: "Device"}
_LIBS: dict = {}


def _reduce(ann):
    """annotation -> (base type, is_list, is_optional)."""
    if isinstance(ann, str):
        raise TypeError(f"string annotation {ann!r}: resolve it first (typing.get_type_hints)")
    origin, args = typing.get_origin(ann), typing.get_args(ann)
    if origin in (typing.Union, types.UnionType):
        rest = [a for a in args if a is not type(None)]
        if len(rest) != 1 or len(rest) == len(args):
            raise TypeError(f"only unions of one type with None are supported, got {ann}")
        base, is_list, _ = _reduce(rest[0])
        return base, is_list, True
    if origin in (list, typing.List, tuple, typing.Sequence) or (
            origin is not None and isinstance(origin, type) and issubclass(origin, (list, tuple, Sequence))):
        inner = [a for a in args if a is not Ellipsis]
        if not inner or any(a is not inner[0] for a in inner):
            raise TypeError(f"homogeneous sequences only, got {ann}")
        base, nested, opt = _reduce(inner[0])
        if nested or opt:
            raise TypeError(f"nested sequences and sequences of optionals are not supported: {ann}")
        return base, True, False
    if ann in _BASE:
        return ann, False, False
    raise TypeError(f"unsupported annotation {ann}")


def _arg_type(ann, mutated: bool) -> str:
    base, is_list, is_opt = _reduce(ann)
    s = _BASE[base]
    if mutated:
        if base is not torch.Tensor:
            raise TypeError("only Tensor arguments can be mutated")
        s += "(a!)"
    return s + ("[]" if is_list else "") + ("?" if is_opt else "")


def _default(v) -> str:
    if v is None:
        return "None"
    if isinstance(v, bool):
        return "True" if v else "False"
    if isinstance(v, str):
        return '"' + v.replace('"', '\\"') + '"'
    if isinstance(v, (int, float)):
        return repr(v)
    if isinstance(v, (list, tuple)) and all(isinstance(e, (int, float)) for e in v):
        return "[" + ", ".join(repr(e) for e in v) + "]"
    raise TypeError(f"default value {v!r} has no schema spelling")


def _return_type(ann) -> str:
    if ann is None or ann is type(None) or ann is inspect.Signature.empty:
        return "()"
    if typing.get_origin(ann) in (tuple, typing.Tuple):
        parts = [a for a in typing.get_args(ann) if a is not Ellipsis]
        if Ellipsis in typing.get_args(ann):
            return "Tensor[]" if parts == [torch.Tensor] else _raise_ret(ann)
        return "(" + ", ".join(_arg_type(p, False) for p in parts) + ")"
    return _arg_type(ann, False)


def _raise_ret(ann):
    raise TypeError(f"unsupported return annotation {ann}")


def infer_schema(fn: Callable, mutates_args: Sequence[str] = ()) -> str:
    """``(Tensor(a!) out, Tensor x, SymInt[]? shape=None, float eps=1e-06) -> ()`` for an annotated function.

    Each mutated Tensor gets its own alias letter; keyword-only parameters are printed after ``*``."""
    hints = typing.get_type_hints(fn)
    sig = inspect.signature(fn)
    unknown = set(mutates_args) - set(sig.parameters)
    if unknown:
        raise ValueError(f"mutates_args names no parameter: {sorted(unknown)}")
    parts, star, letter = [], False, iter("abcdefghijklmnopqrstuvwxyz")
    for name, p in sig.parameters.items():
        if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            raise TypeError("*args / **kwargs have no schema")
        if name not in hints:
            raise TypeError(f"parameter {name!r} of {fn.__name__} is not annotated")
        if p.kind is p.KEYWORD_ONLY and not star:
            parts.append("*")
            star = True
        t = _arg_type(hints[name], name in mutates_args)
        if name in mutates_args:
            t = t.replace("(a!)", f"({next(letter)}!)")
        parts.append(f"{t} {name}" + ("" if p.default is p.empty else f"={_default(p.default)}"))
    return "(" + ", ".join(parts) + ") -> " + _return_type(hints.get("return", sig.return_annotation))


def _library(ns: str) -> "torch.library.Library":
    if ns not in _LIBS:
        _LIBS[ns] = torch.library.Library(ns, "FRAGMENT")
    return _LIBS[ns]


def direct_register_custom_op(op_name: str, op_func: Callable, mutates_args: Sequence[str] = (),
                              fake_impl: Optional[Callable] = None, namespace: str = "b200",
                              dispatch_key: str = "CompositeExplicitAutograd", tags: tuple = ()):
    """Define ``torch.ops.<namespace>.<op_name>`` with the schema of ``op_func`` and return the op.

    ``CompositeExplicitAutograd`` serves every device with the same function (the kernels here pick CPU oracles or
    CUDA themselves); pass ``"CUDA"`` to bind one backend only.  ``fake_impl`` gives output shapes to tracers."""
    lib = _library(namespace)
    lib.define(op_name + infer_schema(op_func, mutates_args), tags=tags)
    lib.impl(op_name, op_func, dispatch_key)
    if fake_impl is not None:
        lib._register_fake(op_name, fake_impl)
    return getattr(getattr(torch.ops, namespace), op_name)
