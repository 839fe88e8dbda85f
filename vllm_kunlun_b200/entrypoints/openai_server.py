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
import logging
import queue
import threading
import time
import uuid
from typing import Optional

from ..engine.request import SamplingParams
from ..multimodal import (InternImagePreprocessor, QwenImagePreprocessor, collect_images, expand_placeholders,
                          load_image)


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

    def stream_delta(self, text: str, fin: Optional[str]):
        """The ``delta`` object of a streamed chat chunk for the next piece of generated text, and the finish reason
        to report (``tool_calls`` when the model called tools).  Reasoning is split off first; the remaining content
        goes through the tool-call scanner: text outside calls stays content, calls stream as OpenAI tool-call deltas
        (the name first, then pieces of the arguments JSON)."""
        delta: dict = {}
        harmony = getattr(self.reasoning, "handles_tools", False)   # the parser reports tool calls of the same stream
        if text or (harmony and fin is not None):
            if self.reasoning is not None:
                d = (self.reasoning.extract_reasoning_streaming(text, final=fin is not None) if harmony
                     else self.reasoning.extract_reasoning_streaming(text))
                if d is not None:
                    if d.reasoning:
                        delta["reasoning_content"] = d.reasoning
                    if d.content:
                        delta["content"] = d.content
                    calls = []
                    for e in (getattr(d, "tool_events", None) or []):
                        if "name" in e:
                            calls.append({"index": e["index"], "id": e["id"], "type": "function",
                                          "function": {"name": e["name"], "arguments": ""}})
                        else:
                            calls.append({"index": e["index"], "function": {"arguments": e["arguments"]}})
                    if calls:
                        delta["tool_calls"] = calls
            else:
                delta["content"] = text
        if harmony and fin is not None and fin != "length" and self.reasoning.tools_called:
            fin = "tool_calls"
        if self.tool is not None:
            content_in = delta.pop("content", "")
            events = self.tool.feed(content_in, self.tools) if content_in else []
            if fin is not None:
                events = events + self.tool.finish()
            content = "".join(e["content"] for e in events if "content" in e)
            calls = []
            for e in events:
                if "name" in e:
                    calls.append({"index": e["index"], "id": e["id"], "type": "function",
                                  "function": {"name": e["name"], "arguments": ""}})
                elif "arguments" in e:
                    calls.append({"index": e["index"], "function": {"arguments": e["arguments"]}})
            if content:
                delta["content"] = content
            if calls:
                delta["tool_calls"] = calls
            if fin is not None and fin != "length" and self.tool.tools_called:
                fin = "tool_calls"
        return delta, fin

    def finalize(self, text: str) -> dict:
        reasoning, content = (None, text)
        calls = []
        if getattr(self.reasoning, "handles_tools", False):
            reasoning, content, calls = self.reasoning.extract_all(text)
        elif self.reasoning is not None:
            reasoning, content = self.reasoning.extract_reasoning(text)
        msg = {"role": "assistant", "content": content}
        if reasoning:
            msg["reasoning_content"] = reasoning
        if calls:
            msg["tool_calls"] = [{"id": cid, "type": "function", "function": {"name": name, "arguments": args}}
                                 for cid, name, args in calls]
        if self.tool is not None and content:
            ex = self.tool.extract_tool_calls(content, self.tools)
            if ex.tools_called:
                msg["content"] = ex.content
                msg["tool_calls"] = [{"id": c.id, "type": "function",
                                      "function": {"name": c.name, "arguments": c.arguments}} for c in ex.tool_calls]
        return msg


class StopStrings:
    """Incremental stop-string matching on decoded text: ``feed`` returns the text that is safe to emit (nothing
    that could still turn out to be the beginning of a stop string) and whether a stop string was reached; the
    stop string itself is never emitted (OpenAI ``stop`` semantics)."""

    def __init__(self, stops=()):
        self.stops = [s for s in stops if s]
        self.hold = max((len(s) for s in self.stops), default=1) - 1
        self.buf = ""

    def feed(self, text: str):
        if not self.stops:
            return text, False
        self.buf += text
        at = min((i for i in (self.buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if at >= 0:
            out, self.buf = self.buf[:at], ""
            return out, True
        keep = min(self.hold, len(self.buf))
        out, self.buf = self.buf[:len(self.buf) - keep], self.buf[len(self.buf) - keep:]
        return out, False

    def flush(self) -> str:
        out, self.buf = self.buf, ""
        return out


def stop_list(body) -> tuple:
    st = body.get("stop")
    return () if not st else ((st,) if isinstance(st, str) else tuple(st))


log = logging.getLogger("vllm_kunlun_b200.server")
try:
    from ..engine.runner import DeviceWaitTimeout
    DEVICE_ERRORS: tuple = (DeviceWaitTimeout,)
except Exception:  # pragma: no cover
    DEVICE_ERRORS = ()


class EngineLoop:
    """Owns the engine on a worker thread.

    With several ranks (one process per GPU, SPMD engine) rank 0 takes the HTTP requests and, once per loop
    iteration, broadcasts the batch of new requests over a gloo control group; every rank then adds the same
    requests and takes the same engine step, so the ranks' schedulers stay identical.  The other ranks call
    :meth:`run_follower` instead of serving HTTP.  The control group is separate from the NCCL groups so that a
    control message never waits on, or syncs with, the GPU streams."""

    def __init__(self, llm, start: bool = True):
        import torch.distributed as dist
        self.llm = llm
        self.inbox: "queue.Queue" = queue.Queue()
        self.streams: dict = {}
        self.stats = {"requests": 0, "tokens": 0, "aborted": 0, "failed": 0}
        self.healthy = True  # cleared when a step failed with a device error (wrong data may be in the caches)
        self._stop = False
        self.aborts: "queue.Queue" = queue.Queue()
        self.multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        self.rank = dist.get_rank() if self.multi else 0
        self.ctrl = dist.new_group(backend="gloo") if self.multi else None  # collective: every rank creates it
        self.thread = None
        if start and self.rank == 0:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def submit(self, prompt_ids, sp: SamplingParams, loop, out_q, lora_id: int = -1, mm: Optional[dict] = None):
        """``mm``: the request's ``multi_modal_data`` (host tensors), or None."""
        rid = f"cmpl-{uuid.uuid4().hex}"
        self.inbox.put((rid, prompt_ids, sp, loop, out_q, lora_id, mm))
        return rid

    def abort(self, rid: str):
        """Ask the loop to drop a request (stop string matched, client gone); takes effect before the next step."""
        self.aborts.put(rid)

    def stop(self):
        """Ends the loop (and, through the last control message, the followers)."""
        self._stop = True
        if self.thread is not None:
            self.thread.join(timeout=30)

    def _broadcast(self, msg):
        import torch.distributed as dist
        box = [msg]
        dist.broadcast_object_list(box, src=0, group=self.ctrl)
        return box[0]

    def run_follower(self):
        """Ranks > 0: mirror rank 0's requests and steps until it says stop."""
        eng = self.llm.engine
        while True:
            kind, new, aborts = self._broadcast(None)
            if kind == "stop":
                return
            for rid in aborts:
                eng.abort(rid)
            for rid, ids, sp, lora_id, mm in new:
                try:
                    eng.add_request(ids, sp, request_id=rid, eos_token_id=self.llm.eos_token_id, lora_id=lora_id,
                                    multi_modal_data=mm)
                except Exception:  # rank 0 validated the request; a failure here is reported there as well
                    log.exception("follower: add_request failed for %s", rid)
            if eng.has_unfinished():
                try:
                    eng.step()
                except Exception:  # rank 0 hits the same failure in its own step and fails the streams
                    log.exception("follower: engine step failed; dropping all requests")
                    eng.abort_all()

    def _run(self):
        eng = self.llm.engine
        sent: dict = {}
        while not self._stop:
            new = []
            try:
                while True:
                    new.append(self.inbox.get_nowait() if (eng.has_unfinished() or new)
                               else self.inbox.get(timeout=0.05))
            except queue.Empty:
                pass
            aborts = []
            while not self.aborts.empty():
                aborts.append(self.aborts.get_nowait())
            if self.multi:
                self._broadcast(("step", [(rid, ids, sp, lora_id, mm) for rid, ids, sp, _, _, lora_id, mm in new], aborts))
            for rid in aborts:
                self.stats["aborted"] += int(eng.abort(rid))
            for rid, ids, sp, loop, out_q, lora_id, mm in new:
                try:
                    req = eng.add_request(ids, sp, request_id=rid, eos_token_id=self.llm.eos_token_id, lora_id=lora_id,
                                          multi_modal_data=mm)
                except Exception as e:  # an unservable request fails alone; the loop and the other streams go on
                    loop.call_soon_threadsafe(out_q.put_nowait, ("error", f"{type(e).__name__}: {e}"))
                    self.stats["failed"] = self.stats.get("failed", 0) + 1
                    continue
                self.streams[rid] = (req, loop, out_q)
                sent[rid] = 0
                self.stats["requests"] += 1
            if eng.has_unfinished():
                try:
                    eng.step()
                except Exception as e:
                    # A failed step (device-side wait time-out, an internal error) must not kill this thread: /health
                    # would keep answering while every request hangs.  Fail the requests that were in the engine, free
                    # their blocks and keep serving.
                    log.exception("engine step failed; failing %d active request(s)", len(self.streams))
                    self.healthy = not isinstance(e, DEVICE_ERRORS)
                    eng.abort_all()
                    for rid, (req, loop, out_q) in list(self.streams.items()):
                        loop.call_soon_threadsafe(out_q.put_nowait, ("error", f"engine step failed: {type(e).__name__}: {e}"))
                        del self.streams[rid], sent[rid]
                    self.stats["failed"] = self.stats.get("failed", 0) + 1
                    continue
            elif not aborts:
                continue
            for rid, (req, loop, out_q) in list(self.streams.items()):
                n = len(req.output_token_ids)
                if n > sent[rid]:
                    new_toks = req.output_token_ids[sent[rid]:n]
                    self.stats["tokens"] += len(new_toks)
                    sent[rid] = n
                    if req.sampling.logprobs:   # log p of every new token, ahead of the tokens themselves
                        loop.call_soon_threadsafe(out_q.put_nowait, ("logprobs", list(req.output_logprobs[n - len(new_toks):n])))
                    loop.call_soon_threadsafe(out_q.put_nowait, ("tokens", new_toks))
                if req.status.finished:
                    reason = "length" if req.status.name.endswith("LENGTH") else "stop"
                    loop.call_soon_threadsafe(out_q.put_nowait, ("done", reason))
                    del self.streams[rid], sent[rid]
        if self.multi:
            self._broadcast(("stop", [], []))


def build_app(llm, model_name: str, reasoning_parser=None, tool_parser=None, lora_modules: Optional[dict] = None):
    """``lora_modules``: adapter name -> adapter id of adapters already loaded with ``llm.add_lora``; a request
    whose ``model`` field names one runs with that adapter (upstream's ``--lora-modules`` convention)."""
    from fastapi import FastAPI, Request
    lora_modules = dict(lora_modules or {})
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI()
    # image inputs: models with a Qwen-VL tower (patch / merge geometry in the configuration) take image_url parts
    vision = getattr(llm.engine.cfg.model, "vision", None) or {}
    pre_cfg = getattr(llm, "preprocessor_config", None)
    if vision.get("layer_scale") and vision.get("image_size"):          # InternViT tower: tiles + thumbnail
        image_pre = InternImagePreprocessor.from_config(vision, pre_cfg)
    elif vision.get("merge") and vision.get("temporal_patch"):
        image_pre = QwenImagePreprocessor.from_config(vision, pre_cfg)
    else:
        image_pre = None
    image_token_id = vision.get("image_token_id")
    loop_obj = EngineLoop(llm)
    app.state.engine_loop = loop_obj
    tok = llm.tokenizer

    def encode(text):
        if tok is None:
            return [int(x) for x in text.split()] if isinstance(text, str) else list(text)
        return tok.encode(text)

    def decode(ids):
        return " ".join(map(str, ids)) if tok is None else tok.decode(ids)

    def logprob_block(ids, lps, obj: str):
        """The ``logprobs`` object of a choice for these tokens: the chat form (``content`` entries) or the completions
        form (parallel lists).  Only the sampled token's log-probability is reported (``top_logprobs`` stays empty)."""
        toks = [decode([t]) for t in ids]
        if obj.startswith("chat"):
            return {"content": [{"token": t, "logprob": lp, "bytes": list(t.encode("utf-8")), "top_logprobs": []}
                                for t, lp in zip(toks, lps)]}
        offs, pos = [], 0
        for t in toks:
            offs.append(pos)
            pos += len(t)
        return {"tokens": toks, "token_logprobs": list(lps), "top_logprobs": None, "text_offset": offs}

    def sampling(body):
        """Request body -> SamplingParams, or an error string (answered with HTTP 400)."""
        try:
            mt = body.get("max_tokens") if body.get("max_tokens") is not None else body.get("max_completion_tokens")
            seed = body.get("seed")
            lp = body.get("logprobs")
            return SamplingParams(max_tokens=16 if mt is None else int(mt),
                                  temperature=float(body.get("temperature", 1.0) if body.get("temperature") is not None else 1.0),
                                  top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", 0) or 0),
                                  ignore_eos=bool(body.get("ignore_eos", False)),
                                  stop_token_ids=tuple(int(t) for t in (body.get("stop_token_ids") or ())),
                                  repetition_penalty=float(body.get("repetition_penalty", 1.0)),
                                  seed=None if seed is None else int(seed), logprobs=bool(lp))
        except (TypeError, ValueError) as e:
            return f"invalid sampling parameter: {e}"

    @app.get("/health")
    async def health():
        alive = loop_obj.thread is None or loop_obj.thread.is_alive()
        if not alive or not loop_obj.healthy:
            return PlainTextResponse("engine loop stopped" if not alive else "device error in an earlier step",
                                     status_code=503)
        return PlainTextResponse("ok")

    @app.get("/v1/models")
    async def models():
        data = [{"id": model_name, "object": "model", "owned_by": "vllm_kunlun_b200"}]
        data += [{"id": n, "object": "model", "owned_by": "vllm_kunlun_b200", "parent": model_name}
                 for n in lora_modules]
        return {"object": "list", "data": data}

    @app.get("/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    @app.post("/tokenize")
    async def tokenize(req: Request):
        """``{"prompt": text}`` or ``{"messages": [...]}`` -> token ids (upstream's helper endpoint)."""
        body = await req.json()
        if "messages" in body and tok is not None and hasattr(tok, "apply_chat_template"):
            ids = tok.apply_chat_template(body["messages"], add_generation_prompt=bool(body.get("add_generation_prompt", True)),
                                          **(body.get("chat_template_kwargs") or {}))
            ids = ids["input_ids"] if hasattr(ids, "keys") else ids
        else:
            ids = encode(body.get("prompt", ""))
        ids = list(ids)
        return {"tokens": ids, "count": len(ids), "max_model_len": llm.engine.cfg.scheduler.max_model_len}

    @app.post("/detokenize")
    async def detokenize(req: Request):
        body = await req.json()
        try:
            ids = [int(t) for t in body.get("tokens", [])]
        except (TypeError, ValueError):
            return bad_request("tokens must be a list of integers")
        return {"prompt": decode(ids)}

    @app.get("/metrics")
    async def metrics():
        s, e = loop_obj.stats, llm.engine.stats
        lines = [f"b200_requests_total {s['requests']}", f"b200_generation_tokens_total {s['tokens']}",
                 f"b200_requests_aborted_total {s['aborted']}",
                 f"b200_engine_steps_total {e['steps']}", f"b200_preemptions_total {e['preemptions']}",
                 f"b200_spec_accepted_total {e['spec_accepted']}", f"b200_spec_proposed_total {e['spec_proposed']}"]
        return PlainTextResponse("\n".join(lines) + "\n")

    def bad_request(msg: str, code: int = 400):
        kind = "BadRequestError" if code == 400 else "InternalServerError"
        return JSONResponse({"error": {"message": msg, "type": kind, "code": code}}, status_code=code)

    async def run(prompt_ids, sp, stream, make_chunk, make_final, requested_model=None, stops=(), mm=None):
        if isinstance(sp, str):  # the sampling parameters did not parse
            return bad_request(sp)
        # the name selects an adapter; with no adapters loaded every name is served by the base model
        if lora_modules and requested_model not in (None, "", model_name) and requested_model not in lora_modules:
            return JSONResponse({"error": {"message": f"The model `{requested_model}` does not exist.",
                                           "type": "NotFoundError", "code": 404}}, status_code=404)
        try:
            llm.engine.validate_request(prompt_ids, sp)
        except ValueError as e:
            return bad_request(str(e))
        loop = asyncio.get_running_loop()
        out_q: asyncio.Queue = asyncio.Queue()
        rid = loop_obj.submit(prompt_ids, sp, loop, out_q, lora_modules.get(requested_model, -1), mm)
        created = int(time.time())
        cut = StopStrings(stops)
        if stream:
            async def gen():
                ids = []
                lps = None
                try:
                    while True:
                        kind, val = await out_q.get()
                        if kind == "logprobs":
                            lps = val
                        elif kind == "tokens":
                            ids += val
                            piece, hit = cut.feed(decode(val))
                            if piece or lps:
                                ch = make_chunk(rid, created, piece, None)
                                if lps:     # the tokens of this step (their text may still be held back by a stop string)
                                    ch["choices"][0]["logprobs"] = logprob_block(val, lps, ch["object"])
                                    lps = None
                                yield f"data: {json.dumps(ch)}\n\n"
                            if hit:
                                loop_obj.abort(rid)
                                yield f"data: {json.dumps(make_chunk(rid, created, '', 'stop'))}\n\n"
                                yield "data: [DONE]\n\n"
                                return
                        elif kind == "error":
                            yield f"data: {json.dumps({'error': {'message': val, 'type': 'InternalServerError', 'code': 500}})}\n\n"
                            yield "data: [DONE]\n\n"
                            return
                        else:
                            rest = cut.flush()
                            if rest:
                                yield f"data: {json.dumps(make_chunk(rid, created, rest, None))}\n\n"
                            yield f"data: {json.dumps(make_chunk(rid, created, '', val))}\n\n"
                            yield "data: [DONE]\n\n"
                            return
                except asyncio.CancelledError:  # the client went away: free the request's blocks
                    loop_obj.abort(rid)
                    raise
            return StreamingResponse(gen(), media_type="text/event-stream")
        ids, reason, text, all_lps = [], None, "", []
        while reason is None:
            kind, val = await out_q.get()
            if kind == "logprobs":
                all_lps += val
            elif kind == "tokens":
                ids += val
                if stops:
                    piece, hit = cut.feed(decode(val))
                    text += piece
                    if hit:
                        loop_obj.abort(rid)
                        reason = "stop"
            elif kind == "error":
                return bad_request(val, 500)
            else:
                reason = val
                text += cut.flush()
        out = make_final(rid, created, text if stops else decode(ids), reason, len(prompt_ids), len(ids))
        if all_lps:
            out["choices"][0]["logprobs"] = logprob_block(ids[:len(all_lps)], all_lps, out["object"])
        return JSONResponse(out)

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
        return await run(ids, sampling(body), bool(body.get("stream")), chunk, final, body.get("model"), stop_list(body))

    @app.post("/v1/chat/completions")
    async def chat(req: Request):
        body = await req.json()
        msgs = body.get("messages", [])
        urls = collect_images(msgs)
        if urls and image_pre is None:
            return bad_request("this model takes no image input")
        if tok is not None and hasattr(tok, "apply_chat_template"):
            ids = tok.apply_chat_template(msgs, add_generation_prompt=True, tools=body.get("tools"),
                                          **(body.get("chat_template_kwargs") or {}))
            ids = ids["input_ids"] if hasattr(ids, "keys") else ids
        else:
            ids = []
            for m in msgs:      # no tokenizer: text parts are lists of ids, every image part is one placeholder
                c = m.get("content", "")
                for part in (c if isinstance(c, list) else [{"type": "text", "text": c}]):
                    if isinstance(part, dict) and ("image_url" in part or part.get("type") in ("image", "image_url")):
                        ids.append(image_token_id)
                    else:
                        ids += encode(str(part.get("text", "")) if isinstance(part, dict) else str(part))
        mm = None
        if urls:
            try:
                px, grids = image_pre([load_image(u) for u in urls])
                ids = expand_placeholders(list(ids), image_token_id, [image_pre.tokens_per_image(g) for g in grids])
            except (ValueError, OSError) as e:
                return bad_request(f"image input: {e}")
            mm = image_pre.mm_data(px, grids)
        post = ChatPostProcessor(reasoning_parser, tool_parser, body.get("tools"), body.get("chat_template_kwargs"))

        def chunk(rid, created, text, fin):
            delta, fin = post.stream_delta(text, fin)
            return {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}

        def final(rid, created, text, fin, n_in, n_out):
            msg = post.finalize(text)
            return {"id": rid, "object": "chat.completion", "created": created, "model": model_name,
                    "choices": [{"index": 0, "message": msg,
                                 "finish_reason": "tool_calls" if msg.get("tool_calls") else fin}],
                    "usage": {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out}}
        return await run(list(ids), sampling(body), bool(body.get("stream")), chunk, final, body.get("model"),
                         stop_list(body), mm)

    return app


def make_parser() -> argparse.ArgumentParser:
    """The flags of upstream's ``vllm serve`` that this engine implements, under the same names."""
    ap = argparse.ArgumentParser(prog="vllm-kunlun-b200 serve")
    ap.add_argument("--model", required=True, help="HF directory or a preset name")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--dtype", default=None, choices=[None, "bfloat16", "float16", "float32"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    ap.add_argument("--pipeline-parallel-size", "-pp", type=int, default=1)
    ap.add_argument("--decode-context-parallel-size", "-dcp", type=int, default=1)
    ap.add_argument("--enable-expert-parallel", action="store_true")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-gpu-blocks-override", type=int, default=None)
    ap.add_argument("--kv-cache-dtype", default="auto")
    ap.add_argument("--enable-prefix-caching", action=argparse.BooleanOptionalAction, default=False)
    ap.add_argument("--enable-chunked-prefill", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--speculative-config", type=json.loads, default=None,
                    help='JSON, e.g. \'{"method": "mtp", "num_speculative_tokens": 1}\'')
    ap.add_argument("--enable-lora", action="store_true")
    ap.add_argument("--max-loras", type=int, default=4)
    ap.add_argument("--max-lora-rank", type=int, default=16)
    ap.add_argument("--lora-modules", nargs="*", default=[], metavar="NAME=PATH",
                    help="adapters to load at start; also JSON objects with name / path keys")
    ap.add_argument("--reasoning-parser", default=None)
    ap.add_argument("--tool-call-parser", default=None)
    ap.add_argument("--enable-auto-tool-choice", action="store_true", help="accepted for compatibility")
    ap.add_argument("--trust-remote-code", action="store_true", help="accepted for compatibility; never executed")
    return ap


def llm_kwargs(a: argparse.Namespace) -> dict:
    """Parsed flags -> keyword arguments of :class:`vllm_kunlun_b200.engine.llm.LLM`."""
    return dict(tensor_parallel_size=a.tensor_parallel_size, pipeline_parallel_size=a.pipeline_parallel_size,
                decode_context_parallel_size=a.decode_context_parallel_size,
                enable_expert_parallel=a.enable_expert_parallel, dtype=a.dtype, seed=a.seed,
                max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
                max_num_batched_tokens=a.max_num_batched_tokens, block_size=a.block_size,
                gpu_memory_utilization=a.gpu_memory_utilization, num_gpu_blocks=a.num_gpu_blocks_override,
                kv_cache_dtype=a.kv_cache_dtype, enable_prefix_caching=a.enable_prefix_caching,
                enable_chunked_prefill=a.enable_chunked_prefill, enforce_eager=a.enforce_eager,
                speculative_config=a.speculative_config, enable_lora=a.enable_lora or bool(a.lora_modules),
                max_loras=max(a.max_loras, len(a.lora_modules)), max_lora_rank=a.max_lora_rank)


def parse_lora_modules(items) -> list:
    """``NAME=PATH`` or ``{"name": ..., "path": ...}`` -> ``[(name, path)]`` in order, names unique."""
    out, seen = [], set()
    for it in items or []:
        if it.lstrip().startswith("{"):
            d = json.loads(it)
            name, path = d["name"], d["path"]
        else:
            name, sep, path = it.partition("=")
            if not sep or not name or not path:
                raise ValueError(f"--lora-modules wants NAME=PATH, got {it!r}")
        if name in seen:
            raise ValueError(f"adapter name {name!r} given twice")
        seen.add(name)
        out.append((name, path))
    return out


def main(argv=None):
    a = make_parser().parse_args(argv)
    import os

    import uvicorn

    from ..engine.llm import LLM
    tokenizer = None
    if os.path.isdir(a.model):
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(a.model)
        except Exception:
            tokenizer = None
    llm = LLM(a.model, tokenizer=tokenizer, **llm_kwargs(a))
    pre = os.path.join(a.model, "preprocessor_config.json")
    if os.path.isfile(pre):     # pixel budget and normalisation statistics of the checkpoint's image processor
        with open(pre) as f:
            llm.preprocessor_config = json.load(f)
    lora_ids = {}
    if a.lora_modules:
        from ..lora import LoRARequest
        for i, (name, path) in enumerate(parse_lora_modules(a.lora_modules), start=1):
            llm.add_lora(LoRARequest(name, i, lora_path=path))
            lora_ids[name] = i
    graphs = llm.engine.runner.graphs
    if graphs is not None:  # capture every decode batch size before the first request arrives
        graphs.capture_all()
    if int(os.environ.get("RANK", "0")) > 0:  # SPMD follower: no HTTP, mirror rank 0
        EngineLoop(llm).run_follower()
        return
    app = build_app(llm, a.served_model_name or a.model, a.reasoning_parser, a.tool_call_parser, lora_ids)
    try:
        uvicorn.run(app, host=a.host, port=a.port, log_level="info")
    finally:
        app.state.engine_loop.stop()


if __name__ == "__main__":
    main()
