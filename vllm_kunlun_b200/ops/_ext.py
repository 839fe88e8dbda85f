"""Loader for the in-tree sm_100a extension ``vllm_kunlun_b200/_C*.so``.

The reference loads its native module ``_kunlun`` at plugin registration
(``vllm_kunlun/__init__.py:76-86``) and silently continues without it.  Here a CUDA tensor reaching
an op without the extension is an error: a GPU run must never fall back to eager PyTorch unnoticed.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import threading

_LOCK = threading.Lock()
_MOD = None
_TRIED = False
_ERR = None

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def so_path():
    cands = sorted(glob.glob(os.path.join(PKG_DIR, "_C*.so")))
    return cands[0] if cands else None


def load(required: bool = False):
    """Return the extension module, or None when it has not been built (CPU-only use)."""
    global _MOD, _TRIED, _ERR
    if _MOD is not None:
        return _MOD
    with _LOCK:
        if _MOD is None and not _TRIED:
            _TRIED = True
            path = so_path()
            if path is not None:
                try:
                    import torch  # noqa: F401  (libtorch symbols must be loaded first)
                    spec = importlib.util.spec_from_file_location("vllm_kunlun_b200._C", path)
                    mod = importlib.util.module_from_spec(spec)
                    spec.loader.exec_module(mod)
                    _MOD = mod
                    _alias_weak_ref_tensor()
                except Exception as e:  # pragma: no cover - depends on the build
                    _ERR = e
            else:
                _ERR = FileNotFoundError(f"no _C*.so under {PKG_DIR}; run `python -m vllm_kunlun_b200.build`")
    if _MOD is None and required:
        raise RuntimeError(f"vllm_kunlun_b200 CUDA extension is not available: {_ERR!r}")
    return _MOD


_LIB = []


def _alias_weak_ref_tensor() -> None:
    """``torch.ops._C.weak_ref_tensor`` is the name upstream's graph capture looks up; define it on top of
    ``_C_b200::weak_ref_tensor`` unless an installed vLLM has already defined it."""
    import torch
    try:
        if hasattr(torch.ops._C, "weak_ref_tensor"):
            return
    except Exception:
        pass
    try:
        lib = torch.library.Library("_C", "FRAGMENT")
        lib.define("weak_ref_tensor(Tensor input) -> Tensor")
        lib.impl("weak_ref_tensor", lambda t: torch.ops._C_b200.weak_ref_tensor(t), "CUDA")
        _LIB.append(lib)
    except Exception:  # defined concurrently by another library: theirs serves
        pass


def C():
    """The extension, required (raises if missing)."""
    return load(required=True)


def available() -> bool:
    return load(False) is not None
