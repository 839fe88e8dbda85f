"""GLM-4.7 tool-call parser: XML-ish model output -> OpenAI ``tool_calls`` with JSON arguments.

Model output format (reference: ``entrypoints/openai/tool_parsers/glm47_moe_tool_parser.py:273-286``)::

    <tool_call>function_name
    <arg_key>k1</arg_key><arg_value>v1</arg_value>
    <arg_key>k2</arg_key><arg_value>v2</arg_value></tool_call>

Argument values are converted according to the tool's JSON schema when one is given (strings stay
strings, numbers / booleans / objects / arrays are parsed), else by best effort.  The streaming
interface re-parses the accumulated text and emits deltas: the function name once it is complete
(an ``<arg_key`` or the closing tag has been seen), then argument JSON text as values complete."""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

TOOL_START, TOOL_END = "<tool_call>", "</tool_call>"
_CALL_RE = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)
_PAIR_RE = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.DOTALL)


@dataclass
class ToolCall:
    name: str
    arguments: str  # JSON text
    id: str = field(default_factory=lambda: f"call_{uuid.uuid4().hex[:24]}")
    type: str = "function"


@dataclass
class ExtractedToolCalls:
    tools_called: bool
    tool_calls: list
    content: Optional[str]


def _schema_type(tools, func: str, key: str) -> Optional[str]:
    for t in tools or []:
        fn = t.get("function", t) if isinstance(t, dict) else getattr(t, "function", t)
        name = fn.get("name") if isinstance(fn, dict) else getattr(fn, "name", None)
        if name != func:
            continue
        params = fn.get("parameters") if isinstance(fn, dict) else getattr(fn, "parameters", None)
        spec = ((params or {}).get("properties") or {}).get(key)
        if not isinstance(spec, dict):
            return None
        ty = spec.get("type")
        if isinstance(ty, list):
            ty = next((x for x in ty if x != "null"), None)
        if ty is None and ("anyOf" in spec or "oneOf" in spec):
            for alt in spec.get("anyOf", spec.get("oneOf", [])):
                if isinstance(alt, dict) and alt.get("type") not in (None, "null"):
                    return alt["type"]
        return ty
    return None


def convert_value(raw: str, ty: Optional[str]) -> Any:
    text = raw.strip()
    if ty == "string":
        return raw if raw == text else text
    if ty in ("integer", "number"):
        try:
            f = float(text)
            return int(f) if (ty == "integer" or f.is_integer() and "." not in text and "e" not in text.lower()) else f
        except ValueError:
            return text
    if ty == "boolean":
        return text.lower() in ("true", "1", "yes")
    if ty in ("object", "array", None):
        try:
            return json.loads(text)
        except (ValueError, TypeError):
            return text
    return text


class Glm47ToolParser:
    def __init__(self, tokenizer=None):
        self._sent_name: list = []      # per streamed call: name already emitted
        self._sent_args: list = []      # per streamed call: argument text already emitted
        self._ids: list = []

    def _parse_call(self, body: str, tools) -> Optional[ToolCall]:
        head, _, rest = body.partition("<arg_key>")
        name = head.strip().split("\n")[0].strip()
        if not name:
            return None
        args = {}
        for k, v in _PAIR_RE.findall(("<arg_key>" + rest) if rest else ""):
            key = k.strip()
            args[key] = convert_value(v, _schema_type(tools, name, key))
        return ToolCall(name=name, arguments=json.dumps(args, ensure_ascii=False))

    def extract_tool_calls(self, model_output: str, tools=None) -> ExtractedToolCalls:
        if TOOL_START not in model_output:
            return ExtractedToolCalls(False, [], model_output)
        calls = [c for c in (self._parse_call(b, tools) for b in _CALL_RE.findall(model_output)) if c]
        content = model_output[: model_output.find(TOOL_START)].strip() or None
        return ExtractedToolCalls(bool(calls), calls, content)

    # ---- streaming ----
    def extract_tool_calls_streaming(self, current_text: str, tools=None) -> list:
        """Returns delta dicts ``{"index", "id"?, "name"?, "arguments"?}`` or ``{"content": ...}``."""
        deltas = []
        starts = [m.start() for m in re.finditer(re.escape(TOOL_START), current_text)]
        for idx, st in enumerate(starts):
            end = current_text.find(TOOL_END, st)
            body = current_text[st + len(TOOL_START): end if end >= 0 else len(current_text)]
            complete = end >= 0
            while len(self._sent_name) <= idx:
                self._sent_name.append(False)
                self._sent_args.append("")
                self._ids.append(f"call_{uuid.uuid4().hex[:24]}")
            name_part, has_key, rest = body.partition("<arg_key")
            if not self._sent_name[idx] and (has_key or complete) and name_part.strip():
                self._sent_name[idx] = True
                deltas.append({"index": idx, "id": self._ids[idx], "name": name_part.strip().split("\n")[0].strip()})
            if not self._sent_name[idx]:
                continue
            name = name_part.strip().split("\n")[0].strip()
            args = {}
            for k, v in _PAIR_RE.findall("<arg_key" + rest if has_key else ""):
                args[k.strip()] = convert_value(v, _schema_type(tools, name, k.strip()))
            text = json.dumps(args, ensure_ascii=False)
            if not complete:
                text = text[:-1] if args else ""  # keep the object open until the call closes
            if len(text) > len(self._sent_args[idx]) and text.startswith(self._sent_args[idx]):
                deltas.append({"index": idx, "arguments": text[len(self._sent_args[idx]):]})
                self._sent_args[idx] = text
        return deltas
