"""gpt-oss ("harmony") output format: channels -> reasoning / content / tool calls, complete and streaming.

A gpt-oss completion is a sequence of messages, each ``<|channel|>NAME[ to=RECIPIENT][ <|constrain|>json]<|message|>BODY``
closed by ``<|end|>`` (more messages follow after ``<|start|>assistant``), ``<|return|>`` (the answer is complete) or
``<|call|>`` (the model calls a tool and stops).  Channel ``analysis`` is the chain of thought, ``final`` the answer,
``commentary`` with a recipient ``functions.NAME`` a tool call whose body is the arguments JSON, and ``commentary``
without a recipient a preamble shown to the user.  The reference serves this format through upstream's harmony
parser inside its forked chat generator (``vllm_kunlun/entrypoints/openai/serving_chat.py:69-76,246-259``); here
one text scanner does it for the bundled server: it is fed text increments of any size (a marker may be split
anywhere) and emits events as soon as text is safe to classify.

The scanner plays both parser roles of ``entrypoints/openai_server.py::ChatPostProcessor``: the reasoning parser
(``--reasoning-parser gpt_oss``) splits analysis from the rest, and - because tool calls are part of the same
stream - it also reports them, so no separate ``--tool-call-parser`` is needed for this family."""
from __future__ import annotations

import uuid
from dataclasses import dataclass
from typing import Optional

START, CHANNEL, MESSAGE, CONSTRAIN = "<|start|>", "<|channel|>", "<|message|>", "<|constrain|>"
END, RETURN, CALL = "<|end|>", "<|return|>", "<|call|>"
_CLOSERS = (END, RETURN, CALL)
_MARKERS = (START, CHANNEL, MESSAGE, CONSTRAIN, END, RETURN, CALL)


@dataclass
class DeltaMessage:
    reasoning: Optional[str] = None
    content: Optional[str] = None
    tool_events: Optional[list] = None      # [{"index", "id", "name"} | {"index", "arguments"}]


def _held_back(buf: str) -> int:
    """Characters at the end of ``buf`` that could be the beginning of a marker."""
    best = 0
    for tag in _MARKERS:
        for n in range(min(len(tag) - 1, len(buf)), 0, -1):
            if buf.endswith(tag[:n]):
                best = max(best, n)
                break
    return best


class HarmonyScanner:
    """``feed(text)`` -> events ``{"reasoning": s}``, ``{"content": s}``, ``{"index": i, "id": .., "name": ..}``,
    ``{"index": i, "arguments": s}``."""

    def __init__(self):
        self.buf = ""
        self.mode = "probe"         # probe | header | body
        self.kind = "content"       # what the current body is: reasoning | content | tool
        self.calls: list = []       # [(id, name, [argument pieces])]
        self.saw_marker = False

    def _open_body(self, header: str, ev: list):
        """``header`` = the text between <|channel|> and <|message|>."""
        head = header.split(CONSTRAIN)[0].strip()
        name, _, rest = head.partition(" ")
        recipient = ""
        for part in rest.split():
            if part.startswith("to="):
                recipient = part[3:]
        if name == "analysis":
            self.kind = "reasoning"
        elif recipient.startswith("functions."):
            self.kind = "tool"
            cid = f"call_{uuid.uuid4().hex[:24]}"
            self.calls.append((cid, recipient[len("functions."):], []))
            ev.append({"index": len(self.calls) - 1, "id": cid, "name": recipient[len("functions."):]})
        else:
            self.kind = "content"   # final, or a commentary preamble
        self.mode = "body"

    def _emit(self, text: str, ev: list):
        if not text:
            return
        if self.kind == "tool":
            self.calls[-1][2].append(text)
            key, item = "arguments", {"index": len(self.calls) - 1, "arguments": text}
        else:
            key, item = self.kind, {self.kind: text}
        if ev and key in ev[-1] and "name" not in ev[-1] and ev[-1].get("index") == item.get("index"):
            ev[-1][key] += text
        else:
            ev.append(item)

    def feed(self, text: str) -> list:
        self.buf += text
        ev: list = []
        while True:
            b = self.buf
            if self.mode == "probe":
                # before the first marker: a template may have put <|channel|> in the prompt, or the model does not
                # speak harmony at all - plain text is content
                pos = min((p for p in (b.find(m) for m in (CHANNEL, START, MESSAGE)) if p >= 0), default=-1)
                if pos < 0:
                    keep = _held_back(b)
                    self.kind = "content"
                    self._emit(b[:len(b) - keep], ev)
                    self.buf = b[len(b) - keep:]
                    break
                self.kind = "content"
                self._emit(b[:pos], ev)
                self.buf = b[pos:]
                self.mode = "header"
                continue
            if self.mode == "header":
                p = b.find(MESSAGE)
                if p < 0:
                    break
                head = b[:p]
                c = head.rfind(CHANNEL)
                self._open_body(head[c + len(CHANNEL):] if c >= 0 else "final", ev)
                self.buf = b[p + len(MESSAGE):]
                continue
            # body
            pos, tag = min(((p, t) for p, t in ((b.find(t), t) for t in _CLOSERS + (START,)) if p >= 0),
                           default=(-1, None))
            if pos < 0:
                keep = _held_back(b)
                self._emit(b[:len(b) - keep], ev)
                self.buf = b[len(b) - keep:]
                break
            self._emit(b[:pos], ev)
            self.buf = b[pos + (len(tag) if tag != START else 0):]
            self.mode = "header"
        return ev

    def finish(self) -> list:
        ev: list = []
        if self.mode in ("probe", "body") and self.buf:
            self._emit(self.buf, ev)
        self.buf = ""
        return ev


class GptOssReasoningParser:
    """Reasoning-parser interface of the bundled server, plus the tool calls found in the same stream."""

    handles_tools = True

    def __init__(self, tokenizer=None, chat_template_kwargs: Optional[dict] = None, **_):
        self._scanner = HarmonyScanner()

    # ---- whole output ----
    def extract_reasoning(self, model_output: str, request=None):
        r, c, _ = self.extract_all(model_output)
        return r, c

    def extract_all(self, model_output: str):
        """(reasoning or None, content or None, [(id, name, arguments JSON text)])."""
        sc = HarmonyScanner()
        events = sc.feed(model_output) + sc.finish()
        reasoning = "".join(e["reasoning"] for e in events if "reasoning" in e)
        content = "".join(e["content"] for e in events if "content" in e)
        calls = [(cid, name, "".join(parts).strip() or "{}") for cid, name, parts in sc.calls]
        return (reasoning or None), (content or None), calls

    # ---- streaming ----
    def extract_reasoning_streaming(self, delta_text: str, final: bool = False) -> Optional[DeltaMessage]:
        events = self._scanner.feed(delta_text) + (self._scanner.finish() if final else [])
        if not events:
            return None
        r = "".join(e["reasoning"] for e in events if "reasoning" in e)
        c = "".join(e["content"] for e in events if "content" in e)
        tools = [e for e in events if "index" in e]
        return DeltaMessage(reasoning=r or None, content=c or None, tool_events=tools or None)

    @property
    def tools_called(self) -> bool:
        return bool(self._scanner.calls)

    def is_reasoning_end(self, text: str) -> bool:
        return (CHANNEL + "final") in text
