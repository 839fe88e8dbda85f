"""The GLM-4.7 tool-call parser as an upstream ``ToolParser`` (``vllm serve --tool-call-parser glm47``).

The reference ships its parser as a file for ``--tool-parser-plugin``
(``entrypoints/openai/tool_parsers/glm47_moe_tool_parser.py:264``); here the class is registered with upstream's
``ToolParserManager`` when the plugin is loaded, so the name is available without a plugin path.  The class is built
lazily because importing upstream's protocol modules is slow and only needed under ``vllm serve``."""
from __future__ import annotations

from .glm47 import TOOL_START, Glm47Scanner

_CLS = None


def build_vllm_tool_parser():
    """Returns the ``ToolParser`` subclass (importing vLLM on first use)."""
    global _CLS
    if _CLS is not None:
        return _CLS
    from vllm.entrypoints.openai.engine.protocol import (DeltaFunctionCall, DeltaMessage, DeltaToolCall,
                                                         ExtractedToolCallInformation, FunctionCall, ToolCall)
    from vllm.tool_parsers.abstract_tool_parser import ToolParser

    def _tools_of(request):
        tools = getattr(request, "tools", None) or []
        return [t.model_dump() if hasattr(t, "model_dump") else t for t in tools]

    class Glm47VllmToolParser(ToolParser):
        def __init__(self, tokenizer, *args, **kwargs):
            super().__init__(tokenizer, *args, **kwargs)
            self._scanner = None

        def extract_tool_calls(self, model_output, request):
            if TOOL_START not in model_output:
                return ExtractedToolCallInformation(tools_called=False, tool_calls=[], content=model_output)
            sc = Glm47Scanner(_tools_of(request))
            events = sc.feed(model_output) + sc.finish()
            calls = [ToolCall(id=cid, type="function", function=FunctionCall(name=name, arguments="".join(parts) or "{}"))
                     for cid, name, parts in sc.calls if name]
            content = "".join(e["content"] for e in events if "content" in e).strip() or None
            return ExtractedToolCallInformation(tools_called=bool(calls), tool_calls=calls, content=content)

        def extract_tool_calls_streaming(self, previous_text, current_text, delta_text, previous_token_ids,
                                         current_token_ids, delta_token_ids, request):
            if self._scanner is None or not previous_text:
                self._scanner = Glm47Scanner(_tools_of(request))
            content, calls = "", []
            for e in self._scanner.feed(delta_text):
                if "content" in e:
                    content += e["content"]
                elif "name" in e:
                    calls.append(DeltaToolCall(index=e["index"], id=e["id"], type="function",
                                               function=DeltaFunctionCall(name=e["name"], arguments="")))
                else:
                    calls.append(DeltaToolCall(index=e["index"], function=DeltaFunctionCall(arguments=e["arguments"])))
            if not content and not calls:
                return None
            return DeltaMessage(content=content or None, tool_calls=calls)

    _CLS = Glm47VllmToolParser
    return _CLS


def register_with_vllm(name: str = "glm47") -> bool:
    """Registers the parser under ``name`` with upstream's manager; False when vLLM is not importable."""
    try:
        from vllm.tool_parsers.abstract_tool_parser import ToolParserManager
    except Exception:  # noqa: BLE001
        return False
    ToolParserManager.register_module(name, True, build_vllm_tool_parser())
    return True
