"""OpenAI-compatible HTTP server on the standalone engine.

    python -m vllm_kunlun_b200.entrypoints.openai_server --model llama-3.1-8b --port 8000

Endpoints: ``/v1/models``, ``/v1/completions``, ``/v1/chat/completions`` (streaming via SSE), ``/health``,
``/metrics``.  The reference relies on upstream's API server and adds a forked chat-completion generator
with reasoning / tool-call streaming (``vllm_kunlun/entrypoints/openai/serving_chat.py:48,699``); the same
post-processing (reasoning parser, tool parser) is wired here through ``ChatPostProcessor``.

One background thread drives ``LLMEngine.step()``; requests are handed over through a queue and their
tokens stream back through per-request asyncio queues."""

import argparse
import asyncio
import json
import queue
import threading
import time
import uuid
from typing import Optional

from ..engine.request import SamplingParams


class ChatPostProcessor:
    """Splits generated text into reasoning / content / tool calls."""

    def __init__(self, reasoning_parser: Optional[str] = None, tool_parser: Optional[str] = None, tools=None,
                 chat_template_kwargs: Optional[dict] = None):
        self.reasoning = None
        self.tool = None
        self.tools = tools
        if reasoning_parser:
            from ..reasoning import get_reasoning_parser
            self.reasoning = get_reasoning_parser(reasoning_parser)(chat_template_kwargs=chat_template_kwargs)
        if tool_parser:
            from .tool_parsers import TOOL_PARSERS
            self.tool = TOOL_PARSERS[tool_parser]()

    def finalize(self, text: str) -> dict:
        reasoning, content = (None, text)
        if self.reasoning is not None:
            reasoning, content = self.reasoning.extract_reasoning(text)
        msg = {"role": "assistant", "content": content}
        if reasoning:
            msg["reasoning_content"] = reasoning
        if self.tool is not None and content:
            ex = self.tool.extract_tool_calls(content, self.tools)
            if ex.tools_called:
                msg["content"] = ex.content
                msg["tool_calls"] = [{"id": c.id, "type": "function",
                                      "function": {"name": c.name, "arguments": c.arguments}} for c in ex.tool_calls]
        return msg


class EngineLoop:
    """Owns the engine on a worker thread."""

    def __init__(self, llm):
        self.llm = llm
        self.inbox: "queue.Queue" = queue.Queue()
        self.streams: dict = {}
        self.stats = {"requests": 0, "tokens": 0}
        self._stop = False
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def submit(self, prompt_ids, sp: SamplingParams, loop, out_q):
        rid = f"cmpl-{uuid.uuid4().hex}"
        self.inbox.put((rid, prompt_ids, sp, loop, out_q))
        return rid

    def _run(self):
        eng = self.llm.engine
        sent: dict = {}
        while not self._stop:
            try:
                while True:
                    rid, ids, sp, loop, out_q = self.inbox.get_nowait() if eng.has_unfinished() else self.inbox.get(timeout=0.05)
                    req = eng.add_request(ids, sp, request_id=rid, eos_token_id=self.llm.eos_token_id)
                    self.streams[rid] = (req, loop, out_q)
                    sent[rid] = 0
                    self.stats["requests"] += 1
            except queue.Empty:
                pass
            if not eng.has_unfinished():
                continue
            eng.step()
            for rid, (req, loop, out_q) in list(self.streams.items()):
                n = len(req.output_token_ids)
                if n > sent[rid]:
                    new = req.output_token_ids[sent[rid]:n]
                    self.stats["tokens"] += len(new)
                    sent[rid] = n
                    loop.call_soon_threadsafe(out_q.put_nowait, ("tokens", new))
                if req.status.finished:
                    reason = "length" if req.status.name.endswith("LENGTH") else "stop"
                    loop.call_soon_threadsafe(out_q.put_nowait, ("done", reason))
                    del self.streams[rid], sent[rid]


def build_app(llm, model_name: str, reasoning_parser=None, tool_parser=None):
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI()
    loop_obj = EngineLoop(llm)
    tok = llm.tokenizer

    def encode(text):
        if tok is None:
            return [int(x) for x in text.split()] if isinstance(text, str) else list(text)
        return tok.encode(text)

    def decode(ids):
        return " ".join(map(str, ids)) if tok is None else tok.decode(ids)

    def sampling(body) -> SamplingParams:
        return SamplingParams(max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 16),
                              temperature=float(body.get("temperature", 1.0) if body.get("temperature") is not None else 1.0),
                              top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", 0) or 0),
                              ignore_eos=bool(body.get("ignore_eos", False)),
                              repetition_penalty=float(body.get("repetition_penalty", 1.0)))

    @app.get("/health")
    async def health():
        return PlainTextResponse("ok")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "vllm_kunlun_b200"}]}

    @app.get("/metrics")
    async def metrics():
        s, e = loop_obj.stats, llm.engine.stats
        lines = [f"b200_requests_total {s['requests']}", f"b200_generation_tokens_total {s['tokens']}",
                 f"b200_engine_steps_total {e['steps']}", f"b200_preemptions_total {e['preemptions']}",
                 f"b200_spec_accepted_total {e['spec_accepted']}", f"b200_spec_proposed_total {e['spec_proposed']}"]
        return PlainTextResponse("\n".join(lines) + "\n")

    async def run(prompt_ids, sp, stream, make_chunk, make_final):
        loop = asyncio.get_running_loop()
        out_q: asyncio.Queue = asyncio.Queue()
        rid = loop_obj.submit(prompt_ids, sp, loop, out_q)
        created = int(time.time())
        if stream:
            async def gen():
                ids = []
                while True:
                    kind, val = await out_q.get()
                    if kind == "tokens":
                        ids += val
                        yield f"data: {json.dumps(make_chunk(rid, created, decode(val), None))}\n\n"
                    else:
                        yield f"data: {json.dumps(make_chunk(rid, created, '', val))}\n\n"
                        yield "data: [DONE]\n\n"
                        return
            return StreamingResponse(gen(), media_type="text/event-stream")
        ids, reason = [], None
        while reason is None:
            kind, val = await out_q.get()
            if kind == "tokens":
                ids += val
            else:
                reason = val
        return JSONResponse(make_final(rid, created, decode(ids), reason, len(prompt_ids), len(ids)))

    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        prompt = body.get("prompt", "")
        ids = encode(prompt) if not (isinstance(prompt, list) and prompt and isinstance(prompt[0], int)) else prompt

        def chunk(rid, created, text, fin):
            return {"id": rid, "object": "text_completion", "created": created, "model": model_name,
                    "choices": [{"index": 0, "text": text, "finish_reason": fin}]}

        def final(rid, created, text, fin, n_in, n_out):
            d = chunk(rid, created, text, fin)
            d["usage"] = {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out}
            return d
        return await run(ids, sampling(body), bool(body.get("stream")), chunk, final)

    @app.post("/v1/chat/completions")
    async def chat(req: Request):
        body = await req.json()
        msgs = body.get("messages", [])
        if tok is not None and hasattr(tok, "apply_chat_template"):
            ids = tok.apply_chat_template(msgs, add_generation_prompt=True, tools=body.get("tools"),
                                          **(body.get("chat_template_kwargs") or {}))
        else:
            ids = encode(" ".join(str(m.get("content", "")) for m in msgs))
        post = ChatPostProcessor(reasoning_parser, tool_parser, body.get("tools"), body.get("chat_template_kwargs"))

        def chunk(rid, created, text, fin):
            delta = {}
            if text:
                if post.reasoning is not None:
                    d = post.reasoning.extract_reasoning_streaming(text)
                    if d is not None:
                        if d.reasoning:
                            delta["reasoning_content"] = d.reasoning
                        if d.content:
                            delta["content"] = d.content
                else:
                    delta["content"] = text
            return {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}

        def final(rid, created, text, fin, n_in, n_out):
            msg = post.finalize(text)
            return {"id": rid, "object": "chat.completion", "created": created, "model": model_name,
                    "choices": [{"index": 0, "message": msg,
                                 "finish_reason": "tool_calls" if msg.get("tool_calls") else fin}],
                    "usage": {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out}}
        return await run(list(ids), sampling(body), bool(body.get("stream")), chunk, final)

    return app


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--reasoning-parser", default=None)
    ap.add_argument("--tool-call-parser", default=None)
    ap.add_argument("--served-model-name", default=None)
    a = ap.parse_args(argv)
    import uvicorn

    from ..engine.llm import LLM
    tokenizer = None
    import os
    if os.path.isdir(a.model):
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(a.model)
        except Exception:
            tokenizer = None
    llm = LLM(a.model, tensor_parallel_size=a.tensor_parallel_size, max_model_len=a.max_model_len,
              max_num_seqs=a.max_num_seqs, block_size=a.block_size, gpu_memory_utilization=a.gpu_memory_utilization,
              enforce_eager=a.enforce_eager, tokenizer=tokenizer)
    graphs = llm.engine.runner.graphs
    if graphs is not None:  # capture every decode batch size before the first request arrives
        graphs.capture_all()
    app = build_app(llm, a.served_model_name or a.model, a.reasoning_parser, a.tool_call_parser)
    uvicorn.run(app, host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
