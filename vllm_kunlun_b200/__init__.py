"""vllm_kunlun_b200: a Blackwell (sm_100a) inference framework with the capabilities of the
vLLM-Kunlun plugin.

Two ways in:

* standalone - ``from vllm_kunlun_b200 import LLM, SamplingParams`` (own scheduler, paged KV cache,
  CUDA-graph runner, OpenAI-compatible server in :mod:`vllm_kunlun_b200.entrypoints`);
* as a vLLM out-of-tree platform plugin - the entry points below have the names and return
  conventions of the reference (``vllm_kunlun/__init__.py:114-150``): ``register`` returns the
  platform class path, ``register_model`` / ``register_reasoning_parser`` / ``register_quant_method``
  are general plugins.  Unlike the reference, registration installs no ``builtins.__import__`` hook
  and patches no upstream file.
"""
from __future__ import annotations

from .version import __version__  # noqa: F401

_completed_steps: set = set()


def register() -> str:
    """``vllm.platform_plugins`` entry point."""
    if "native" not in _completed_steps:
        from .ops import _ext
        _ext.load(required=False)
        _completed_steps.add("native")
    return "vllm_kunlun_b200.platforms.b200.B200Platform"


def register_model() -> None:
    """``vllm.general_plugins`` entry point: expose this package's architectures to upstream's
    ``ModelRegistry`` when vLLM is importable."""
    if "model" in _completed_steps:
        return
    _completed_steps.add("model")
    from .platforms.b200 import register_models_with_vllm
    register_models_with_vllm()


def register_reasoning_parser() -> None:
    if "reasoning" in _completed_steps:
        return
    _completed_steps.add("reasoning")
    from .reasoning import register_reasoning_parsers
    register_reasoning_parsers()


def register_tool_parser() -> None:
    """``vllm.general_plugins`` entry point: the GLM-4.7 tool-call parser under upstream's ``--tool-call-parser glm47``
    (the reference ships the parser as a file for ``--tool-parser-plugin``)."""
    if "tool_parser" in _completed_steps:
        return
    _completed_steps.add("tool_parser")
    from .entrypoints.tool_parsers.vllm_adapter import register_with_vllm
    register_with_vllm()


def register_quant_method() -> None:
    if "quant" in _completed_steps:
        return
    _completed_steps.add("quant")
    from . import quantization  # noqa: F401
    from .quantization.vllm_registry import register_quant_configs
    register_quant_configs()


def register_custom_ops() -> None:
    """``vllm.general_plugins`` entry point: define the ``torch.ops.b200.*`` dispatcher ops for tracing hosts."""
    from .ops.custom_ops import register_custom_ops as _reg
    _reg()
    from .ops.oot_layers import register_oot_layers
    register_oot_layers()


def __getattr__(name):
    if name in ("LLM", "LLMEngine", "SamplingParams", "RequestOutput"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
