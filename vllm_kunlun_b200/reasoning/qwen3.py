"""Qwen3 / Qwen3.5 ``<think> ... </think>`` reasoning parser.

Behaviour of the reference parser (``vllm_kunlun/reasoning/qwen3_reasoning_parser.py:16-151``):
newer chat templates put ``<think>`` in the prompt so only ``</think>`` appears in the output; older
ones let the model emit ``<think>`` itself (it is stripped).  With thinking enabled (default) an output
without ``</think>`` is all reasoning (truncated); with ``enable_thinking=False`` it is all content."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class DeltaMessage:
    reasoning: Optional[str] = None
    content: Optional[str] = None


class Qwen3ReasoningParser:
    start_token = "<think>"
    end_token = "</think>"

    def __init__(self, tokenizer=None, chat_template_kwargs: Optional[dict] = None, **_):
        self.thinking_enabled = (chat_template_kwargs or {}).get("enable_thinking", True)
        self._buf = ""       # streamed text not yet classified (may hold a partial tag)
        self._in_reasoning = self.thinking_enabled
        self._seen_end = False

    # ---- whole-output ----
    def extract_reasoning(self, model_output: str, request=None):
        head, sep, tail = model_output.partition(self.start_token)
        text = tail if sep else head
        if self.end_token not in text:
            return (text, None) if self.thinking_enabled else (None, text)
        reasoning, _, content = text.partition(self.end_token)
        return reasoning, (content or None)

    # ---- streaming ----
    def extract_reasoning_streaming(self, delta_text: str) -> Optional[DeltaMessage]:
        """Feed the next text delta; returns what can be emitted now (or None while a tag is split)."""
        self._buf += delta_text
        out_r, out_c = "", ""
        while self._buf:
            if not self._in_reasoning:
                out_c += self._buf
                self._buf = ""
                break
            # drop a leading <think> emitted by older templates
            if self._buf.startswith(self.start_token):
                self._buf = self._buf[len(self.start_token):]
                continue
            i = self._buf.find(self.end_token)
            if i >= 0:
                out_r += self._buf[:i]
                self._buf = self._buf[i + len(self.end_token):]
                self._in_reasoning = False
                self._seen_end = True
                continue
            # keep a possible partial tag at the end of the buffer
            keep = 0
            for tag in (self.end_token, self.start_token):
                for n in range(min(len(tag) - 1, len(self._buf)), 0, -1):
                    if self._buf.endswith(tag[:n]):
                        keep = max(keep, n)
                        break
            emit = self._buf[:len(self._buf) - keep] if keep else self._buf
            out_r += emit
            self._buf = self._buf[len(emit):]
            break
        if not out_r and not out_c:
            return None
        return DeltaMessage(reasoning=out_r or None, content=out_c or None)

    def is_reasoning_end(self, text: str) -> bool:
        return self.end_token in text
