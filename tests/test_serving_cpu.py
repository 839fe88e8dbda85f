"""Reasoning parser, tool parser, plugin entry points, platform, env registry, loader, utils."""
import json

import pytest
import os

import torch

import vllm_kunlun_b200 as pkg
from vllm_kunlun_b200.entrypoints.tool_parsers import Glm47ToolParser
from vllm_kunlun_b200.reasoning import Qwen3ReasoningParser


def test_qwen3_reasoning_whole_and_streaming():
    p = Qwen3ReasoningParser()
    assert p.extract_reasoning("<think>abc</think>xyz") == ("abc", "xyz")
    assert p.extract_reasoning("abc</think>xyz") == ("abc", "xyz")
    assert p.extract_reasoning("still thinking") == ("still thinking", None)
    assert Qwen3ReasoningParser(chat_template_kwargs={"enable_thinking": False}).extract_reasoning("hi") == (None, "hi")
    s = Qwen3ReasoningParser()
    r, c = "", ""
    for piece in ["<thi", "nk>rea", "son</th", "ink>ans", "wer"]:
        d = s.extract_reasoning_streaming(piece)
        if d:
            r += d.reasoning or ""
            c += d.content or ""
    assert (r, c) == ("reason", "answer")


_WEATHER_TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"},
                                     "opts": {"type": "object"}, "note": {"type": ["string", "null"]},
                                     "unit": {"enum": ["C", "F"]}, "when": {"anyOf": [{"type": "integer"}, {"type": "string"}]},
                                     "tags": {"items": {"type": "string"}}, "flag": {"type": "boolean"}}}}}]


def test_glm47_tool_parser():
    tools = _WEATHER_TOOLS
    out = ("I will call.<tool_call>get_weather\n<arg_key>city</arg_key><arg_value>Paris</arg_value>"
           "<arg_key>days</arg_key><arg_value>3</arg_value>\n<arg_key>opts</arg_key>"
           "<arg_value>{\"units\": \"C\"}</arg_value></tool_call>")
    p = Glm47ToolParser()
    ex = p.extract_tool_calls(out, tools)
    assert ex.tools_called and ex.content == "I will call."
    assert ex.tool_calls[0].name == "get_weather"
    assert json.loads(ex.tool_calls[0].arguments) == {"city": "Paris", "days": 3, "opts": {"units": "C"}}
    assert ex.tool_calls[0].arguments == json.dumps({"city": "Paris", "days": 3, "opts": {"units": "C"}})
    assert not p.extract_tool_calls("no tools here").tools_called
    # streaming: name first, then argument text that concatenates to the final JSON
    sp = Glm47ToolParser()
    name, args = None, ""
    for i in range(1, len(out) + 1, 7):
        for d in sp.extract_tool_calls_streaming(out[:i], tools):
            name = d.get("name", name)
            args += d.get("arguments", "")
    for d in sp.extract_tool_calls_streaming(out, tools):
        args += d.get("arguments", "")
    assert name == "get_weather" and json.loads(args) == {"city": "Paris", "days": 3, "opts": {"units": "C"}}


def test_glm47_schema_types():
    from vllm_kunlun_b200.entrypoints.tool_parsers.glm47 import argument_type, convert_value, infer_schema_type
    t = _WEATHER_TOOLS
    assert [argument_type(t, "get_weather", k) for k in ("city", "days", "opts", "note", "unit", "when", "tags", "flag")] == \
        ["string", "integer", "object", "string", "string", "string", "array", "boolean"]
    assert argument_type(t, "get_weather", "missing") is None and argument_type(t, "other", "city") is None
    assert infer_schema_type({"anyOf": [{"type": "integer"}, {"type": "null"}]}) == "integer"
    assert infer_schema_type({"enum": [1, 2]}) == "integer" and infer_schema_type({"enum": [1, "a"]}) == "string"
    assert infer_schema_type({"allOf": [{"type": "string"}, {"type": "object"}]}) == "object"
    assert infer_schema_type({"properties": {}}) == "object" and infer_schema_type({}) is None
    assert convert_value("3", "integer") == 3 and convert_value("2.5", "number") == 2.5 and convert_value("7", "number") == 7
    assert convert_value("True", "boolean") is True and convert_value("no", "boolean") is False
    assert convert_value("{'a': True}", "object") == {"a": True}            # python-literal spelling
    assert convert_value("[1, 2]", None) == [1, 2] and convert_value("plain", None) == "plain"
    assert convert_value("12x", "integer") == "12x"


def test_glm47_streaming_any_split_multiple_calls_and_string_values_flow():
    """Whatever the split of the text into increments: the events rebuild the same calls; a string value is forwarded
    before its closing tag arrives; text around calls stays content; a call without arguments gives ``{}``; a call the
    model never closed is closed at the end of the stream."""
    from vllm_kunlun_b200.entrypoints.tool_parsers.glm47 import Glm47Scanner
    text = ("Let me check. <tool_call>get_weather\n<arg_key>city</arg_key><arg_value>San \"Quoted\" José\nline2</arg_value>"
            "<arg_key>flag</arg_key><arg_value>true</arg_value><arg_key>tags</arg_key><arg_value>[\"a\", \"b\"]</arg_value>"
            "</tool_call>\n<tool_call>ping</tool_call> done <not a tag> "
            "<tool_call>get_weather\n<arg_key>city</arg_key><arg_value>Oslo")
    want = [("get_weather", {"city": "San \"Quoted\" José\nline2", "flag": True, "tags": ["a", "b"]}), ("ping", {}),
            ("get_weather", {"city": "Oslo"})]

    def run(step):
        sc = Glm47Scanner(_WEATHER_TOOLS)
        events = []
        for i in range(0, len(text), step):
            events += sc.feed(text[i:i + step])
        events += sc.finish()
        names, args, content = {}, {}, ""
        for e in events:
            if "content" in e:
                content += e["content"]
            else:
                if "name" in e:
                    names[e["index"]] = e["name"]
                    assert e["id"].startswith("call_")
                args[e["index"]] = args.get(e["index"], "") + e.get("arguments", "")
        return [(names[i], json.loads(args[i])) for i in sorted(names)], content, events

    for step in (1, 2, 3, 5, 11, 64, len(text)):
        calls, content, _ = run(step)
        assert calls == want, step
        assert content == "Let me check. \n done <not a tag> ", (step, content)
    # the string value streams: with one character per increment, argument pieces of call 0 arrive before the closing tag
    sc = Glm47Scanner(_WEATHER_TOOLS)
    seen = ""
    upto = text.index("line2")
    for ch in text[:upto]:
        for e in sc.feed(ch):
            seen += e.get("arguments", "")
    assert seen.startswith('{"city": "San \\"Quoted\\" Jos') and not seen.endswith('"')


def test_chat_stream_delta_assembles_tool_call_chunks():
    from vllm_kunlun_b200.entrypoints.openai_server import ChatPostProcessor
    post = ChatPostProcessor(None, "glm47", _WEATHER_TOOLS)
    text = "ok <tool_call>get_weather\n<arg_key>days</arg_key><arg_value>2</arg_value></tool_call>"
    deltas, fin = [], None
    for i in range(0, len(text), 9):
        d, f = post.stream_delta(text[i:i + 9], None)
        deltas.append(d)
    d, fin = post.stream_delta("", "stop")
    deltas.append(d)
    assert fin == "tool_calls"
    assert "".join(d.get("content", "") for d in deltas) == "ok "
    calls = [c for d in deltas for c in d.get("tool_calls", [])]
    assert calls[0]["function"]["name"] == "get_weather" and calls[0]["type"] == "function" and calls[0]["index"] == 0
    assert json.loads("".join(c["function"]["arguments"] for c in calls)) == {"days": 2}
    # no tool call: content passes through and the finish reason stays
    post = ChatPostProcessor(None, "glm47", _WEATHER_TOOLS)
    d1, _ = post.stream_delta("plain <text", None)
    d2, fin = post.stream_delta("", "stop")
    assert d1.get("content", "") + d2.get("content", "") == "plain <text" and fin == "stop"


def test_plugin_entry_points_and_platform():
    assert pkg.register() == "vllm_kunlun_b200.platforms.b200.B200Platform"
    pkg.register_reasoning_parser()
    pkg.register_quant_method()
    from vllm_kunlun_b200.platforms.b200 import B200Platform
    assert B200Platform.dist_backend == "nccl" and B200Platform.device_type == "cuda"
    assert B200Platform.get_device_communicator_cls().endswith("B200Communicator")
    from types import SimpleNamespace
    assert "MLA" in B200Platform.get_attn_backend_cls(None, SimpleNamespace(use_mla=True, use_sparse=False))
    assert B200Platform.get_device_total_memory() > (1 << 30)

    class _C:  # minimal stand-in for a vLLM config
        class cache_config:
            block_size = None
        class model_config:
            use_mla = True
        compilation_config = None
        parallel_config = None
    B200Platform.check_and_update_config(_C)
    assert _C.cache_config.block_size == 64
    from vllm_kunlun_b200.models import supported_architectures
    archs = supported_architectures()
    for a in ("LlamaForCausalLM", "Qwen3MoeForCausalLM", "DeepseekV32ForCausalLM", "DeepSeekMTPModel", "GptOssForCausalLM"):
        assert a in archs


def test_env_registry_is_lazy(monkeypatch):
    from vllm_kunlun_b200 import envs
    monkeypatch.setenv("B200_PDL", "0")
    assert envs.B200_PDL is False
    monkeypatch.setenv("B200_PDL", "1")
    assert envs.B200_PDL is True
    assert "B200_SPIN_LIMIT" in envs.describe()


def test_safetensors_roundtrip_with_fp8_scales(tmp_path):
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.config import qwen3_30b_a3b, tiny
    from vllm_kunlun_b200.models.loader import load_safetensors, save_safetensors
    cfg = tiny(qwen3_30b_a3b(fp8=True), num_layers=1, vocab_size=128, hidden_size=128, num_heads=2, num_kv_heads=2,
               head_dim=64, intermediate_size=256, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
               max_position=256, dtype="float32")
    a = LLM(cfg, device="cpu", block_size=16, max_model_len=64, max_num_seqs=2, num_gpu_blocks=8)
    # export in checkpoint naming: split fused tensors back into q/k/v, gate/up and per-expert tensors
    m = a.engine.runner.model
    sd = {}
    L = m.layers["0"]
    q, kv = cfg.q_size, cfg.kv_size
    for suffix in ("weight", "weight_scale_inv"):
        t = getattr(L.self_attn.qkv_proj, suffix).data
        div = 128 if suffix == "weight_scale_inv" else 1
        sd[f"model.layers.0.self_attn.q_proj.{suffix}"] = t[: q // div]
        sd[f"model.layers.0.self_attn.k_proj.{suffix}"] = t[q // div:(q + kv) // div]
        sd[f"model.layers.0.self_attn.v_proj.{suffix}"] = t[(q + kv) // div:]
        sd[f"model.layers.0.self_attn.o_proj.{suffix}"] = getattr(L.self_attn.o_proj, suffix).data
    sd["model.layers.0.self_attn.q_norm.weight"] = L.self_attn.q_norm.weight.data
    sd["model.layers.0.self_attn.k_norm.weight"] = L.self_attn.k_norm.weight.data
    sd["model.layers.0.input_layernorm.weight"] = L.input_layernorm.weight.data
    sd["model.layers.0.post_attention_layernorm.weight"] = L.post_attention_layernorm.weight.data
    sd["model.layers.0.mlp.gate.weight"] = L.mlp.gate.weight.data
    ex = L.mlp.experts
    I = ex.i_local
    for e in range(4):
        sd[f"model.layers.0.mlp.experts.{e}.gate_proj.weight"] = ex.w13.data[e, :I]
        sd[f"model.layers.0.mlp.experts.{e}.up_proj.weight"] = ex.w13.data[e, I:]
        sd[f"model.layers.0.mlp.experts.{e}.down_proj.weight"] = ex.w2.data[e]
        sd[f"model.layers.0.mlp.experts.{e}.gate_proj.weight_scale_inv"] = ex.w13_scale.data[e, : I // 128]
        sd[f"model.layers.0.mlp.experts.{e}.up_proj.weight_scale_inv"] = ex.w13_scale.data[e, I // 128:]
        sd[f"model.layers.0.mlp.experts.{e}.down_proj.weight_scale_inv"] = ex.w2_scale.data[e]
    sd["model.embed_tokens.weight"] = m.embed_tokens.weight.data[: cfg.vocab_size]
    sd["model.norm.weight"] = m.norm.weight.data
    sd["lm_head.weight"] = m.lm_head.weight.data[: cfg.vocab_size]
    save_safetensors({k: v.clone() for k, v in sd.items()}, str(tmp_path))
    names = {n for n, _ in load_safetensors(str(tmp_path))}
    assert "model.layers.0.mlp.experts.3.down_proj.weight_scale_inv" in names
    b = LLM(cfg, device="cpu", block_size=16, max_model_len=64, max_num_seqs=2, num_gpu_blocks=8, seed=99)
    with torch.inference_mode():
        b.engine.runner.model.load_weights(load_safetensors(str(tmp_path)))
    prompt = [list(range(3, 20))]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    assert a.generate(prompt, sp)[0].token_ids == b.generate(prompt, sp)[0].token_ids


def test_module_tracer_and_stage_timer():
    from vllm_kunlun_b200.utils import ModuleTracer, StageTimer
    lines = []
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU())
    with ModuleTracer(net, lines.append):
        net(torch.zeros(2, 4))
    assert any("Linear" in l for l in lines) and any("<-" in l for l in lines)
    st = StageTimer(sink=None)
    with st.stage("first token"):
        pass
    assert st.records[0][0] == "first token"


def test_openai_server_completions_and_chat_stream():
    from fastapi.testclient import TestClient

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    app = build_app(llm, "tiny", reasoning_parser="qwen3")
    with TestClient(app) as c:
        assert c.get("/health").text == "ok"
        assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
        assert c.get("/version").json()["version"]
        t = c.post("/tokenize", json={"prompt": "5 6 7"}).json()
        assert t["tokens"] == [5, 6, 7] and t["count"] == 3 and t["max_model_len"] > 0
        assert c.post("/detokenize", json={"tokens": [5, 6, 7]}).json()["prompt"] == "5 6 7"
        assert c.post("/detokenize", json={"tokens": ["x"]}).status_code == 400
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 4, "temperature": 0, "ignore_eos": True})
        body = r.json()
        assert body["usage"]["completion_tokens"] == 4 and body["choices"][0]["finish_reason"] == "length"
        ref = llm_tokens = body["choices"][0]["text"]
        # same request, streamed: the concatenated chunks equal the non-streamed text
        with c.stream("POST", "/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 4, "temperature": 0,
                                                       "ignore_eos": True, "stream": True}) as s:
            pieces = []
            for line in s.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    pieces.append(json.loads(line[6:])["choices"][0]["text"])
        assert " ".join(p for p in pieces if p) == ref
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "1 2 3"}], "max_tokens": 3,
                                                 "temperature": 0, "ignore_eos": True})
        msg = r.json()["choices"][0]["message"]
        assert msg["role"] == "assistant" and "reasoning_content" in msg
        assert "b200_requests_total 3" in c.get("/metrics").text


def test_bench_serving_client_against_live_server():
    """The serving benchmark client drives a real HTTP server (uvicorn on a free port) over the tiny CPU engine."""
    import importlib.util
    import socket
    import threading
    import time

    import uvicorn

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = uvicorn.Server(uvicorn.Config(build_app(llm, "tiny"), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(100):
        if server.started:
            break
        time.sleep(0.1)
    assert server.started
    spec = importlib.util.spec_from_file_location(
        "bench_serving", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "bench_serving.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        out = mod.main(["--port", str(port), "--num-prompts", "4", "--max-concurrency", "2", "--random-input-len", "12",
                        "--random-output-len", "6", "--vocab-size", "100"])
    finally:
        server.should_exit = True
        th.join(timeout=10)
    assert out["completed"] == 4 and out["failed"] == 0 and out["output_tok_per_s"] > 0


class _Sel:
    def __init__(self, use_mla, use_sparse):
        self.use_mla, self.use_sparse = use_mla, use_sparse


def test_platform_class_paths_resolve():
    """Every "module.Class" string the platform hands to an engine imports and names an existing attribute."""
    import importlib

    from vllm_kunlun_b200.platforms.b200 import B200Platform
    paths = [B200Platform.get_device_communicator_cls(), B200Platform.get_punica_wrapper(),
             B200Platform.get_attn_backend_cls(None, None), B200Platform.get_attn_backend_cls(None, _Sel(True, False)),
             B200Platform.get_attn_backend_cls(None, _Sel(True, True)), B200Platform.get_static_graph_wrapper_cls(),
             pkg.register()]
    for p in paths:
        mod, _, name = p.rpartition(".")
        assert hasattr(importlib.import_module(mod), name), p
    for dt in (torch.bfloat16, torch.float8_e4m3fn, torch.int8):
        B200Platform.check_if_supports_dtype(dt)


def test_graph_input_watcher_detects_moved_tensors():
    import pytest

    from vllm_kunlun_b200.utils import GraphInputWatcher
    w = GraphInputWatcher()
    buf = torch.zeros(8)
    w.capture("g", {"ids": buf[:4], "n": 3})
    w.check("g", {"ids": buf[:4]})
    buf[:4].fill_(7)                      # new contents at the same address are what a replay expects
    w.check("g", {"ids": buf[:4]})
    with pytest.raises(RuntimeError):
        w.check("g", {"ids": buf[4:]})    # another address
    with pytest.raises(KeyError):
        w.check("other", {})


def test_serve_flags_map_to_llm_arguments():
    import inspect

    import pytest

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.entrypoints.openai_server import llm_kwargs, make_parser, parse_lora_modules
    a = make_parser().parse_args([
        "--model", "qwen3-30b-a3b", "-tp", "2", "--enable-expert-parallel", "--no-enable-chunked-prefill",
        "--enable-prefix-caching", "--speculative-config", '{"method": "ngram", "num_speculative_tokens": 2}',
        "--lora-modules", "sql=/adapters/sql", '{"name": "chat", "path": "/adapters/chat"}', "--max-loras", "1",
        "--num-gpu-blocks-override", "77", "--kv-cache-dtype", "fp8", "--trust-remote-code"])
    kw = llm_kwargs(a)
    assert set(kw) <= set(inspect.signature(LLM.__init__).parameters)  # every key is a constructor argument
    assert kw["tensor_parallel_size"] == 2 and kw["enable_expert_parallel"] and not kw["enable_chunked_prefill"]
    assert kw["enable_prefix_caching"] and kw["speculative_config"]["method"] == "ngram"
    assert kw["enable_lora"] and kw["max_loras"] == 2 and kw["num_gpu_blocks"] == 77 and kw["kv_cache_dtype"] == "fp8"
    assert parse_lora_modules(a.lora_modules) == [("sql", "/adapters/sql"), ("chat", "/adapters/chat")]
    for bad in (["x"], ["=p"], ["a=1", "a=2"]):
        with pytest.raises(ValueError):
            parse_lora_modules(bad)
    d = llm_kwargs(make_parser().parse_args(["--model", "m"]))
    assert not d["enable_lora"] and d["enable_chunked_prefill"] and d["speculative_config"] is None


def test_openai_server_routes_adapters_by_model_name():
    from fastapi.testclient import TestClient

    from test_lora_cpu import _adapter, _cfg
    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    cfg = _cfg()
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    llm = LLM(cfg, enable_lora=True, max_loras=2, max_lora_rank=8, **kw)
    ad = _adapter(cfg, 1)
    llm.add_lora(ad)
    prompt = list(range(3, 20))
    sp = SamplingParams(max_tokens=6, ignore_eos=True, temperature=0.0)
    want_base = llm.generate([prompt], sp)[0].token_ids
    want_lora = llm.generate([prompt], sp, lora_request=ad)[0].token_ids
    assert want_base != want_lora
    app = build_app(llm, "base", lora_modules={"sql": ad.lora_int_id})
    with TestClient(app) as c:
        assert [m["id"] for m in c.get("/v1/models").json()["data"]] == ["base", "sql"]
        body = {"prompt": prompt, "max_tokens": 6, "temperature": 0.0, "ignore_eos": True}
        got_base = c.post("/v1/completions", json=dict(body, model="base")).json()["choices"][0]["text"]
        got_lora = c.post("/v1/completions", json=dict(body, model="sql")).json()["choices"][0]["text"]
        assert got_base == " ".join(map(str, want_base)) and got_lora == " ".join(map(str, want_lora))
        r = c.post("/v1/completions", json=dict(body, model="nope"))
        assert r.status_code == 404 and "does not exist" in r.json()["error"]["message"]


def test_stop_strings_incremental():
    from vllm_kunlun_b200.entrypoints.openai_server import StopStrings, stop_list
    s = StopStrings(["</end>", "\n\n"])
    out, hit = "", False
    for piece in ["hel", "lo <", "/en", "x <", "/end", ">tail"]:
        p, hit = s.feed(piece)
        out += p
        if hit:
            break
    assert hit and out == "hello </enx "  # a look-alike prefix is released once it cannot match any more
    s = StopStrings(["STOP"])
    assert s.feed("abcST") == ("ab", False) and s.flush() == "cST"  # held-back tail comes out at the end
    assert StopStrings(()).feed("abc") == ("abc", False)
    assert stop_list({}) == () and stop_list({"stop": "a"}) == ("a",) and stop_list({"stop": ["a", "b"]}) == ("a", "b")


def test_openai_server_stop_string_and_stop_token_abort_the_request():
    import json

    from fastapi.testclient import TestClient

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    app = build_app(llm, "tiny")
    body = {"prompt": list(range(5, 17)), "max_tokens": 12, "temperature": 0.0, "ignore_eos": True}
    with TestClient(app) as c:
        toks = [int(t) for t in c.post("/v1/completions", json=body).json()["choices"][0]["text"].split()]
        assert len(toks) == 12
        # a stop token id ends the request inside the engine, at its first occurrence
        r = c.post("/v1/completions", json=dict(body, stop_token_ids=[toks[4]])).json()
        got = [int(t) for t in r["choices"][0]["text"].split()]
        assert got == toks[:toks.index(toks[4]) + 1] and r["choices"][0]["finish_reason"] == "stop"
        # a stop string is matched on the decoded text (without a tokenizer: the ids' digits, one piece per token)
        full = "".join(map(str, toks))
        stop = str(toks[6])
        r = c.post("/v1/completions", json=dict(body, stop=stop)).json()
        assert r["choices"][0]["text"] == full[:full.find(stop)] and r["choices"][0]["finish_reason"] == "stop"
        assert r["usage"]["completion_tokens"] < 12
        # streaming: the same text arrives in pieces and the stream closes with finish_reason stop
        with c.stream("POST", "/v1/completions", json=dict(body, stop=stop, stream=True)) as resp:
            events = [json.loads(l[6:]) for l in resp.iter_lines() if l.startswith("data: {")]
        assert "".join(e["choices"][0]["text"] for e in events) == full[:full.find(stop)]
        assert events[-1]["choices"][0]["finish_reason"] == "stop"
        # the aborted requests released their blocks: a fresh request still runs to its full length
        again = c.post("/v1/completions", json=body).json()["choices"][0]["text"].split()
        assert [int(t) for t in again] == toks
        assert app.state.engine_loop.stats["aborted"] >= 1
    assert not llm.engine.has_unfinished()


def test_openai_server_returns_logprobs_when_asked():
    from fastapi.testclient import TestClient

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    cfg = tiny(qwen2_0_5b(), num_layers=1, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
               intermediate_size=128, max_position=256, dtype="float32")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=32)
    app = build_app(llm, "tiny")
    body = {"prompt": [5, 6, 7, 8], "max_tokens": 5, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        plain = c.post("/v1/completions", json=body).json()
        assert "logprobs" not in plain["choices"][0]
        r = c.post("/v1/completions", json=dict(body, logprobs=1)).json()
        lp = r["choices"][0]["logprobs"]
        assert r["choices"][0]["text"] == plain["choices"][0]["text"]
        assert len(lp["tokens"]) == 5 and " ".join(lp["tokens"]) == r["choices"][0]["text"]
        assert len(lp["token_logprobs"]) == 5 and all(v <= 0.0 for v in lp["token_logprobs"])
        assert lp["text_offset"][0] == 0 and lp["text_offset"] == sorted(lp["text_offset"])
        # greedy: the sampled token is the most likely one, so its probability is at least 1 / vocab
        import math
        assert all(v >= math.log(1 / 128) for v in lp["token_logprobs"])
        chat = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "1 2 3"}], "max_tokens": 3,
                                                    "temperature": 0, "ignore_eos": True, "logprobs": True}).json()
        entries = chat["choices"][0]["logprobs"]["content"]
        assert len(entries) == 3 and all(e["logprob"] <= 0 and e["top_logprobs"] == [] for e in entries)
        # streamed: the chunks carry the same values
        with c.stream("POST", "/v1/completions", json=dict(body, logprobs=1, stream=True)) as s:
            got = []
            for line in s.iter_lines():
                if line.startswith("data: {"):
                    ch = json.loads(line[6:])["choices"][0]
                    got += (ch.get("logprobs") or {}).get("token_logprobs", [])
        assert got == pytest.approx(lp["token_logprobs"], abs=1e-5)


_HARMONY = ("<|channel|>analysis<|message|>The user wants weather. I should call the tool.<|end|>"
            "<|start|>assistant<|channel|>commentary<|message|>Checking the forecast.<|end|>"
            "<|start|>assistant<|channel|>commentary to=functions.get_weather <|constrain|>json<|message|>"
            "{\"city\": \"Paris\", \"days\": 2}<|call|>")
_HARMONY_ANSWER = ("<|channel|>analysis<|message|>Simple sum.<|end|><|start|>assistant<|channel|>final<|message|>"
                   "2 + 2 = 4<|return|>")


def test_gpt_oss_harmony_channels_whole_and_streaming():
    """analysis -> reasoning, final / commentary preamble -> content, commentary to=functions.X -> a tool call whose
    body is the arguments JSON; any split of the stream gives the same result."""
    from vllm_kunlun_b200.reasoning import get_reasoning_parser
    cls = get_reasoning_parser("gpt_oss")
    assert get_reasoning_parser("openai_gptoss") is cls
    r, c, calls = cls().extract_all(_HARMONY)
    assert r == "The user wants weather. I should call the tool." and c == "Checking the forecast."
    assert [(n, json.loads(a)) for _, n, a in calls] == [("get_weather", {"city": "Paris", "days": 2})]
    assert cls().extract_reasoning(_HARMONY_ANSWER) == ("Simple sum.", "2 + 2 = 4")
    assert cls().extract_reasoning("no markers at all") == (None, "no markers at all")
    for step in (1, 2, 3, 7, 16, len(_HARMONY)):
        p = cls()
        r, c, name, args = "", "", None, ""
        for i in range(0, len(_HARMONY), step):
            d = p.extract_reasoning_streaming(_HARMONY[i:i + step], final=i + step >= len(_HARMONY))
            if d is None:
                continue
            r += d.reasoning or ""
            c += d.content or ""
            for e in d.tool_events or []:
                name = e.get("name", name)
                args += e.get("arguments", "")
        assert (r, c, name) == ("The user wants weather. I should call the tool.", "Checking the forecast.", "get_weather"), step
        assert json.loads(args) == {"city": "Paris", "days": 2} and p.tools_called


def test_chat_post_processor_with_harmony_parser():
    from vllm_kunlun_b200.entrypoints.openai_server import ChatPostProcessor
    msg = ChatPostProcessor("gpt_oss").finalize(_HARMONY)
    assert msg["reasoning_content"].startswith("The user wants") and msg["content"] == "Checking the forecast."
    assert msg["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(msg["tool_calls"][0]["function"]["arguments"]) == {"city": "Paris", "days": 2}
    post = ChatPostProcessor("gpt_oss")
    deltas = [post.stream_delta(_HARMONY[i:i + 11], None)[0] for i in range(0, len(_HARMONY), 11)]
    last, fin = post.stream_delta("", "stop")
    deltas.append(last)
    assert fin == "tool_calls"
    assert "".join(d.get("reasoning_content", "") for d in deltas) == "The user wants weather. I should call the tool."
    assert "".join(d.get("content", "") for d in deltas) == "Checking the forecast."
    calls = [c for d in deltas for c in d.get("tool_calls", [])]
    assert calls[0]["function"]["name"] == "get_weather"
    assert json.loads("".join(c["function"]["arguments"] for c in calls)) == {"city": "Paris", "days": 2}
    post = ChatPostProcessor("gpt_oss")
    deltas = [post.stream_delta(_HARMONY_ANSWER[i:i + 5], None)[0] for i in range(0, len(_HARMONY_ANSWER), 5)]
    last, fin = post.stream_delta("", "stop")
    assert fin == "stop" and "".join(d.get("content", "") for d in deltas + [last]) == "2 + 2 = 4"


def test_image_preprocessor_matches_the_transformers_processor():
    """Same grid and patch order as ``Qwen2VLImageProcessor``; pixel values within one intensity level (the two
    bicubic resamplers round differently)."""
    np = pytest.importorskip("numpy")
    transformers = pytest.importorskip("transformers")
    from PIL import Image

    from vllm_kunlun_b200.multimodal import QwenImagePreprocessor, expand_placeholders, smart_resize
    assert smart_resize(37, 91, 28, 56 * 56, 28 * 28 * 64) == (56, 112)
    rng = np.random.default_rng(0)
    mine = QwenImagePreprocessor(14, 2, 2, 56 * 56, 28 * 28 * 64)
    hp = transformers.Qwen2VLImageProcessor(patch_size=14, temporal_patch_size=2, merge_size=2,
                                            size={"shortest_edge": 56 * 56, "longest_edge": 28 * 28 * 64})
    for H, W in ((120, 200), (37, 91), (600, 300)):
        # smooth content: both resamplers agree to rounding (on noise they differ by design)
        yy, xx = np.mgrid[0:H, 0:W]
        arr = np.stack([(yy * 255 // H), (xx * 255 // W), ((yy + xx) * 255 // (H + W))], -1).astype(np.uint8)
        im = Image.fromarray(arr)
        want = hp(images=[im], return_tensors="pt")
        px, grid = mine([im])
        assert grid == want["image_grid_thw"].tolist()
        assert px.shape == want["pixel_values"].shape
        assert (px - want["pixel_values"]).abs().max().item() <= 2.1 / 255 / 0.26
        assert mine.tokens_per_image(grid[0]) == grid[0][1] * grid[0][2] // 4
    assert expand_placeholders([1, 9, 2, 9, 9, 3], 9, [3, 2]) == [1, 9, 9, 9, 2, 9, 9, 3]
    with pytest.raises(ValueError):
        expand_placeholders([1, 9, 2], 9, [3, 2])


def test_openai_server_chat_with_an_image_part():
    """An ``image_url`` part (data: URI) reaches the engine as pixel values + grid with the placeholder expanded; the
    answer depends on the image; a text-only model answers 400."""
    import base64
    import io

    from fastapi.testclient import TestClient
    from PIL import Image

    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.config import qwen2_0_5b, tiny
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    base = dict(num_layers=2, vocab_size=128, hidden_size=64, num_heads=2, num_kv_heads=1, head_dim=32,
                intermediate_size=128, max_position=512, dtype="float32")
    cfg = tiny(qwen2_0_5b(), **base)
    cfg.architecture = "Qwen2VLForConditionalGeneration"
    cfg.mrope_section = (4, 6, 6)
    cfg.vision = dict(depth=1, hidden=32, heads=2, patch=14, temporal_patch=2, merge=2, intermediate=64, in_channels=3,
                      norm="layernorm", gated_mlp=False, image_token_id=127, text_architecture="Qwen2ForCausalLM")
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=64)

    def uri(color):
        buf = io.BytesIO()
        Image.new("RGB", (60, 90), color).save(buf, format="PNG")
        return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

    def ask(c, color):
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "text", "text": "3 4 5"}, {"type": "image_url", "image_url": {"url": uri(color)}},
            {"type": "text", "text": "6 7"}]}], "max_tokens": 6, "temperature": 0, "ignore_eos": True, "logprobs": True})
        assert r.status_code == 200, r.text
        return r.json()

    with TestClient(build_app(llm, "vl")) as c:
        a, b = ask(c, (250, 10, 10)), ask(c, (10, 10, 250))
        # 60 x 90 -> 56 x 84 pixels -> 4 x 6 patches -> 6 placeholder tokens + 5 text tokens
        assert a["usage"]["prompt_tokens"] == 11
        lp = lambda d: [e["logprob"] for e in d["choices"][0]["logprobs"]["content"]]  # noqa: E731
        assert lp(a) != lp(b)
        assert lp(ask(c, (250, 10, 10))) == lp(a)
        bad = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}], "max_tokens": 2})
        assert bad.status_code == 400
    text_llm = LLM(tiny(qwen2_0_5b(), **base), device="cpu", block_size=16, max_model_len=128, max_num_seqs=2, num_gpu_blocks=32)
    with TestClient(build_app(text_llm, "text")) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": uri((1, 2, 3))}}]}], "max_tokens": 2})
        assert r.status_code == 400


def test_openai_server_chat_with_an_image_part_internvl_tiles():
    """InternVL: the image is cut into tiles of the tower's size plus a thumbnail; the single placeholder grows to
    tiles x tokens-per-tile."""
    import base64
    import io
    import sys

    from fastapi.testclient import TestClient
    from PIL import Image

    sys.path.insert(0, os.path.dirname(__file__))
    from test_vision_cpu import _intern
    from vllm_kunlun_b200 import LLM
    from vllm_kunlun_b200.entrypoints.openai_server import build_app
    from vllm_kunlun_b200.multimodal import InternImagePreprocessor
    pre = InternImagePreprocessor(448, 14, 0.5, 1, 12, True)
    assert pre.tile_grid(800, 400) == (2, 1) and pre.tile_grid(448, 448) == (1, 1) and pre.tile_grid(300, 1200) == (1, 4)
    assert pre.tokens_per_tile == 256
    llm = LLM(_intern(), device="cpu", block_size=16, max_model_len=256, max_num_seqs=2, num_gpu_blocks=64)
    buf = io.BytesIO()
    Image.new("RGB", (16, 8), (200, 30, 30)).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    with TestClient(build_app(llm, "intern")) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "text", "text": "3 4"}, {"type": "image_url", "image_url": {"url": uri}}]}],
            "max_tokens": 3, "temperature": 0, "ignore_eos": True})
        assert r.status_code == 200, r.text
        # 16 x 8 pixels on an 8-pixel tower: a 2 x 1 grid of tiles + thumbnail, 4 tokens each, + 2 text tokens
        assert r.json()["usage"]["prompt_tokens"] == 3 * 4 + 2
