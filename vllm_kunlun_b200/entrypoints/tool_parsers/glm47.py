"""GLM-4.7 tool-call parser: XML-ish model output -> OpenAI ``tool_calls`` with JSON arguments, complete and streaming.

Model output format (reference: ``entrypoints/openai/tool_parsers/glm47_moe_tool_parser.py:273-286``)::

    <tool_call>function_name
    <arg_key>k1</arg_key><arg_value>v1</arg_value>
    <arg_key>k2</arg_key><arg_value>v2</arg_value></tool_call>

One scanner serves both interfaces.  It is fed text increments of any size (a tag may be split anywhere) and turns
them into events: plain content, the function name of call ``i`` (as soon as the first ``<arg_key>`` or the closing
tag shows that the name is complete) and pieces of the call's ``arguments`` JSON text.  String-typed values are
forwarded while they are being generated (escaped piece by piece, so a long code or text argument streams like
content does); values of every other type are held until ``</arg_value>`` and then emitted as one JSON value,
converted according to the tool's JSON schema (``type``, type lists, ``anyOf`` / ``oneOf``, ``enum``, ``allOf``,
``properties`` -> object, ``items`` -> array; the reference's rules, ``glm47_moe_tool_parser.py:161-262``) or, without
a schema, by best effort.  The pieces of a call always concatenate to the text ``json.dumps`` gives for the parsed
arguments, and the complete interface is the streaming one run over the whole text, so the two cannot disagree.
``vllm_adapter.py`` wraps the same scanner as an upstream ``ToolParser`` registered under the name ``glm47``."""
from __future__ import annotations

import ast
import json
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

TOOL_START, TOOL_END = "<tool_call>", "</tool_call>"
KEY_START, KEY_END = "<arg_key>", "</arg_key>"
VAL_START, VAL_END = "<arg_value>", "</arg_value>"


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


# ----------------------------------------------------------------------------- schema

def infer_schema_type(schema) -> Optional[str]:
    """The JSON type a schema asks for, or None when it does not say."""
    if not isinstance(schema, dict):
        return None
    ty = schema.get("type")
    if isinstance(ty, str):
        return ty
    if isinstance(ty, list) and ty:
        return next((t for t in ty if t != "null"), "string")
    for comb in ("anyOf", "oneOf"):
        alts = schema.get(comb)
        if isinstance(alts, list):
            kinds = [k for k in (infer_schema_type(a) for a in alts) if k and k != "null"]
            if kinds:
                # one kind: that one; several: a string can hold anything the model wrote
                return kinds[0] if len(set(kinds)) == 1 or "string" not in kinds else "string"
    enum = schema.get("enum")
    if isinstance(enum, list):
        names = {("null" if v is None else "boolean" if isinstance(v, bool) else "integer" if isinstance(v, int)
                  else "number" if isinstance(v, float) else "string" if isinstance(v, str)
                  else "array" if isinstance(v, list) else "object") for v in enum}
        return names.pop() if len(names) == 1 else "string"
    if isinstance(schema.get("allOf"), list):
        for sub in schema["allOf"]:
            k = infer_schema_type(sub)
            if k and k != "string":
                return k
        return "string"
    if "properties" in schema:
        return "object"
    if "items" in schema:
        return "array"
    return None


def _function_spec(tool):
    if isinstance(tool, dict):
        return tool.get("function", tool)
    fn = getattr(tool, "function", tool)
    if hasattr(fn, "model_dump"):
        return fn.model_dump()
    return fn if isinstance(fn, dict) else {"name": getattr(fn, "name", None), "parameters": getattr(fn, "parameters", None)}


def argument_type(tools, func: str, key: str) -> Optional[str]:
    for t in tools or []:
        fn = _function_spec(t)
        if not isinstance(fn, dict) or fn.get("name") != func:
            continue
        params = fn.get("parameters") or {}
        spec = (params.get("properties") or {}).get(key) if isinstance(params, dict) else None
        return infer_schema_type(spec)
    return None


def convert_value(raw: str, ty: Optional[str]) -> Any:
    """The Python value of an ``<arg_value>`` body for a parameter of JSON type ``ty`` (None: unknown)."""
    text = raw.strip()
    if ty == "string":
        return raw if raw == text else text
    if ty in ("integer", "number"):
        try:
            f = float(text)
            whole = f.is_integer() and "." not in text and "e" not in text.lower()
            return int(f) if (ty == "integer" and f.is_integer()) or whole else f
        except (ValueError, OverflowError):
            return text
    if ty == "boolean":
        return text.lower() in ("true", "1", "yes")
    if ty == "null":
        return None
    try:
        return json.loads(text)
    except (ValueError, TypeError):
        pass
    if ty in ("object", "array"):           # python-literal spelling: single quotes, True / None
        try:
            v = ast.literal_eval(text)
            if isinstance(v, (dict, list, tuple)):
                return list(v) if isinstance(v, tuple) else v
        except (ValueError, SyntaxError, MemoryError, RecursionError):
            pass
    return text


# ----------------------------------------------------------------------------- scanner

def _held_back(buf: str, tags) -> int:
    """How many characters at the end of ``buf`` could be the beginning of one of ``tags``."""
    best = 0
    for tag in tags:
        for n in range(min(len(tag) - 1, len(buf)), 0, -1):
            if buf.endswith(tag[:n]):
                best = max(best, n)
                break
    return best


def _first(buf: str, tags):
    """(position, tag) of the earliest of ``tags`` in ``buf``, or (-1, None)."""
    hits = [(p, t) for p, t in ((buf.find(t), t) for t in tags) if p >= 0]
    return min(hits) if hits else (-1, None)


class Glm47Scanner:
    """Incremental converter.  ``feed(text)`` returns events:

    ``{"content": str}`` - text outside tool calls;
    ``{"index": i, "id": str, "name": str}`` - call ``i`` has started and this is its function;
    ``{"index": i, "arguments": str}`` - the next piece of the call's arguments JSON text."""

    def __init__(self, tools=None):
        self.tools = tools
        self.buf = ""
        self.mode = "text"          # text | name | between | key | wait | value
        self.index = -1
        self.name = ""
        self.n_args = 0
        self.key = ""
        self.vtype: Optional[str] = None
        self.raw = ""               # value body collected so far (types other than string)
        self.quote_open = False     # the opening quote of a streamed string value has been emitted
        self.calls: list = []       # [(id, name, [argument pieces])]

    # -- emit helpers
    def _args(self, ev, piece: str):
        if piece:
            self.calls[self.index][2].append(piece)
            if ev and ev[-1].get("index") == self.index and "arguments" in ev[-1] and "name" not in ev[-1]:
                ev[-1]["arguments"] += piece
            else:
                ev.append({"index": self.index, "arguments": piece})

    def _start_call(self, ev, name_text: str):
        lines = name_text.strip().splitlines()
        self.name = lines[0].strip() if lines else ""
        cid = f"call_{uuid.uuid4().hex[:24]}"
        self.calls.append((cid, self.name, []))
        ev.append({"index": self.index, "id": cid, "name": self.name})

    def _close_call(self, ev):
        self._args(ev, "}" if self.n_args else "{}")
        self.mode = "text"

    def feed(self, text: str) -> list:
        self.buf += text
        ev: list = []
        while True:
            b = self.buf
            if self.mode == "text":
                p = b.find(TOOL_START)
                if p >= 0:
                    if b[:p]:
                        ev.append({"content": b[:p]})
                    self.buf = b[p + len(TOOL_START):]
                    self.mode, self.index, self.n_args = "name", self.index + 1, 0
                    continue
                keep = _held_back(b, (TOOL_START,))
                if len(b) > keep:
                    ev.append({"content": b[:len(b) - keep]})
                    self.buf = b[len(b) - keep:]
                break
            if self.mode == "name":
                p, tag = _first(b, (KEY_START, TOOL_END))
                if p < 0:
                    break
                self._start_call(ev, b[:p])
                self.buf = b[p + len(tag):]
                if tag == TOOL_END:
                    self._close_call(ev)
                else:
                    self.mode = "key"
                continue
            if self.mode == "between":
                p, tag = _first(b, (KEY_START, TOOL_END))
                if p < 0:     # only white space is expected here: keep what may be the start of a tag
                    lt = b.find("<")
                    self.buf = b[lt:] if lt >= 0 else ""
                    break
                self.buf = b[p + len(tag):]
                if tag == TOOL_END:
                    self._close_call(ev)
                else:
                    self.mode = "key"
                continue
            if self.mode == "key":
                p = b.find(KEY_END)
                if p < 0:
                    break
                self.key = b[:p].strip()
                self.buf = b[p + len(KEY_END):]
                self._args(ev, ("{" if self.n_args == 0 else ", ") + json.dumps(self.key, ensure_ascii=False) + ": ")
                self.n_args += 1
                self.mode = "wait"
                continue
            if self.mode == "wait":
                p = b.find(VAL_START)
                if p < 0:
                    break
                self.buf = b[p + len(VAL_START):]
                self.vtype = argument_type(self.tools, self.name, self.key)
                self.raw, self.quote_open, self.mode = "", False, "value"
                continue
            # value
            p = b.find(VAL_END)
            body = b[:p] if p >= 0 else b[:len(b) - _held_back(b, (VAL_END,))]
            if self.vtype == "string":
                if body or p >= 0:
                    piece = ("" if self.quote_open else '"') + json.dumps(body, ensure_ascii=False)[1:-1]
                    self.quote_open = True
                    self._args(ev, piece + ('"' if p >= 0 else ""))
            else:
                self.raw += body
                if p >= 0:
                    self._args(ev, json.dumps(convert_value(self.raw, self.vtype), ensure_ascii=False))
            if p >= 0:
                self.buf = b[p + len(VAL_END):]
                self.mode = "between"
                continue
            self.buf = b[len(body):]
            break
        return ev

    def finish(self) -> list:
        """End of the generation: what was held back as a possible tag goes out, and a call that the model did not
        close is closed, so that its arguments are still JSON."""
        ev: list = []
        if self.mode == "text":
            if self.buf:
                ev.append({"content": self.buf})
        elif self.mode == "name":
            if self.buf.strip():
                self._start_call(ev, self.buf)
                self._close_call(ev)
        else:
            if self.mode == "value":
                if self.vtype == "string":
                    self._args(ev, ("" if self.quote_open else '"') + json.dumps(self.buf, ensure_ascii=False)[1:-1] + '"')
                else:
                    self._args(ev, json.dumps(convert_value(self.raw + self.buf, self.vtype), ensure_ascii=False))
            elif self.mode == "wait":
                self._args(ev, "null")
            elif self.mode == "key":
                pass                      # a key that never completed is dropped
            self._close_call(ev)
        self.buf, self.mode = "", "text"
        return ev


class Glm47ToolParser:
    """Complete and streaming extraction for the server (``entrypoints/openai_server.py``)."""

    def __init__(self, tokenizer=None):
        self._scanner: Optional[Glm47Scanner] = None
        self._seen = 0

    def extract_tool_calls(self, model_output: str, tools=None) -> ExtractedToolCalls:
        if TOOL_START not in model_output:
            return ExtractedToolCalls(False, [], model_output)
        sc = Glm47Scanner(tools)
        events = sc.feed(model_output) + sc.finish()
        calls = [ToolCall(name=name, arguments="".join(parts) or "{}", id=cid) for cid, name, parts in sc.calls if name]
        content = "".join(e["content"] for e in events if "content" in e).strip() or None
        return ExtractedToolCalls(bool(calls), calls, content)

    # ---- streaming ----
    def feed(self, delta_text: str, tools=None) -> list:
        """Events for the next piece of generated text (see ``Glm47Scanner``)."""
        if self._scanner is None:
            self._scanner = Glm47Scanner(tools)
        return self._scanner.feed(delta_text)

    def finish(self) -> list:
        return self._scanner.finish() if self._scanner is not None else []

    @property
    def tools_called(self) -> bool:
        return self._scanner is not None and bool(self._scanner.calls)

    def extract_tool_calls_streaming(self, current_text: str, tools=None) -> list:
        """Cumulative-text form: ``current_text`` is everything generated so far."""
        delta, self._seen = current_text[self._seen:], len(current_text)
        return [e for e in self.feed(delta, tools) if "content" not in e]
