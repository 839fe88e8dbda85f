"""Reasoning parsers.  ``register_reasoning_parsers`` registers ``"qwen3"`` with upstream's
``ReasoningParserManager`` when vLLM is importable (the reference does the same,
``vllm_kunlun/reasoning/__init__.py:10-22``); the parsers themselves are dependency-free."""
from .gpt_oss import GptOssReasoningParser
from .qwen3 import Qwen3ReasoningParser

# "gpt_oss" (alias "openai_gptoss", upstream's name) reads the harmony channels: analysis -> reasoning, final ->
# content, commentary to=functions.* -> tool calls
REASONING_PARSERS = {"qwen3": Qwen3ReasoningParser, "gpt_oss": GptOssReasoningParser,
                     "openai_gptoss": GptOssReasoningParser}


def get_reasoning_parser(name: str):
    return REASONING_PARSERS[name]


def register_reasoning_parsers() -> bool:
    try:
        from vllm.reasoning import ReasoningParserManager
    except Exception:
        return False
    try:
        ReasoningParserManager.register_lazy_module("qwen3_b200", "vllm_kunlun_b200.reasoning.qwen3",
                                                    "Qwen3ReasoningParser")
    except Exception:
        try:
            ReasoningParserManager.register_module("qwen3_b200", True, Qwen3ReasoningParser)
        except Exception:
            return False
    return True
