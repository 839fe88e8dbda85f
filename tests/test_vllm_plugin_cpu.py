"""The package as an out-of-tree plugin of the INSTALLED vLLM: entry points are discovered through upstream's own
loader, every class path the platform hands out resolves to a subclass of the installed base with a compatible
signature, and the dense backend's builder / implementation run on upstream's ``CommonAttentionMetadata``."""
import importlib
import inspect
import os
import sys

import pytest
import torch

vllm = pytest.importorskip("vllm")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _resolve(path: str):
    mod, _, name = path.rpartition(".")
    return getattr(importlib.import_module(mod), name)


def _params(fn):
    return [p.name for p in inspect.signature(fn).parameters.values()]


def test_entry_points_load_through_upstreams_plugin_loader():
    from vllm.plugins import load_plugins_by_group
    assert ROOT in sys.path
    plat = load_plugins_by_group("vllm.platform_plugins")
    assert "b200" in plat, f"platform plugin not discovered: {sorted(plat)}"
    assert plat["b200"]() == "vllm_kunlun_b200.platforms.b200.B200Platform"
    general = load_plugins_by_group("vllm.general_plugins")
    for name in ("b200_model", "b200_quant", "b200_ops", "b200_reasoning_parser", "b200_tool_parser"):
        assert name in general, name
        general[name]()  # each registration runs against the installed vLLM


def test_platform_is_an_upstream_platform_with_upstreams_signatures():
    from vllm.platforms.interface import Platform, PlatformEnum
    from vllm_kunlun_b200.platforms.b200 import B200Platform
    assert issubclass(B200Platform, Platform) and B200Platform._enum == PlatformEnum.OOT
    assert B200Platform().is_out_of_tree()
    for name in ("get_attn_backend_cls", "get_device_communicator_cls", "get_punica_wrapper", "check_and_update_config",
                 "get_device_capability", "get_device_total_memory", "check_if_supports_dtype"):
        ours, base = getattr(B200Platform, name), getattr(Platform, name)
        assert _params(ours)[:len(_params(base))] == _params(base), f"{name}: {_params(ours)} vs {_params(base)}"


class _Sel:
    def __init__(self, use_mla=False, use_sparse=False):
        self.use_mla, self.use_sparse = use_mla, use_sparse


def test_backend_selection_follows_the_selector_config():
    from vllm.v1.attention.backend import AttentionBackend
    from vllm_kunlun_b200.platforms.b200 import B200Platform
    got = {}
    for key, sel in (("gqa", _Sel()), ("mla", _Sel(True)), ("sparse", _Sel(True, True))):
        path = B200Platform.get_attn_backend_cls(None, sel, 32)
        cls = _resolve(path)
        assert issubclass(cls, AttentionBackend), path
        got[key] = cls
    assert got["gqa"].__name__ == "GQABackend" and got["mla"].__name__ == "MLABackend"
    assert got["sparse"].__name__ == "SparseMLABackend" and got["sparse"].is_sparse() and got["mla"].is_mla()


def test_backend_quadruple_derives_from_the_installed_bases():
    from vllm.model_executor.layers.attention.mla_attention import MLACommonBackend, MLACommonImpl
    from vllm.v1.attention.backend import AttentionImpl, AttentionMetadataBuilder
    from vllm_kunlun_b200.attention.backends import GQABackend, MLABackend, SparseMLABackend
    impl, builder = GQABackend.get_impl_cls(), GQABackend.get_builder_cls()
    assert issubclass(impl, AttentionImpl) and issubclass(builder, AttentionMetadataBuilder)
    assert _params(impl.forward) == _params(AttentionImpl.forward)
    assert _params(impl.__init__)[:len(_params(AttentionImpl.__init__))] == _params(AttentionImpl.__init__)
    assert _params(builder.__init__) == _params(AttentionMetadataBuilder.__init__)
    assert _params(builder.build) == _params(AttentionMetadataBuilder.build)
    assert GQABackend.get_kv_cache_shape(7, 64, 2, 128) == (7, 2, 2, 64, 128)
    assert GQABackend.get_kv_cache_block_dim(64, 2, 128) == 0
    assert issubclass(MLABackend, MLACommonBackend) and issubclass(MLABackend.get_impl_cls(), MLACommonImpl)
    assert "forward_mqa" in MLABackend.get_impl_cls().__dict__
    assert SparseMLABackend.get_kv_cache_shape(5, 64, 1, 576, "fp8_ds_mla") == (5, 64, 656)


def test_communicator_and_punica_derive_from_upstream_with_upstreams_constructors():
    from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase
    from vllm.lora.punica_wrapper.punica_base import PunicaWrapperBase
    from vllm_kunlun_b200.platforms.b200 import B200Platform
    comm = _resolve(B200Platform.get_device_communicator_cls())
    assert issubclass(comm, DeviceCommunicatorBase)
    assert _params(comm.__init__) == _params(DeviceCommunicatorBase.__init__)
    for m in ("all_reduce", "all_gather", "send", "recv", "destroy"):
        assert _params(getattr(comm, m)) == _params(getattr(DeviceCommunicatorBase, m)), m
    punica = _resolve(B200Platform.get_punica_wrapper())
    assert issubclass(punica, PunicaWrapperBase)
    for m in ("add_shrink", "add_expand", "add_lora_embedding", "add_lora_linear", "add_lora_logits"):
        assert _params(getattr(punica, m)) == _params(getattr(PunicaWrapperBase, m)), m
    assert not inspect.isabstract(punica)


def test_oot_layers_and_quant_config_are_in_upstreams_registries():
    from vllm.model_executor.custom_op import op_registry_oot
    from vllm.model_executor.layers.layernorm import RMSNorm
    from vllm.model_executor.layers.quantization import get_quantization_config
    from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
    from vllm_kunlun_b200.ops.oot_layers import register_oot_layers
    from vllm_kunlun_b200.quantization.vllm_registry import register_quant_configs
    reg = register_oot_layers()
    for name in ("RMSNorm", "GemmaRMSNorm", "SiluAndMul", "RotaryEmbedding", "VocabParallelEmbedding"):
        assert op_registry_oot[name] is reg[name], name
        assert "forward_oot" in reg[name].__dict__ or "forward" in reg[name].__dict__
    assert issubclass(reg["RMSNorm"], RMSNorm)
    from vllm.model_executor.layers import utils as U
    assert U.dispatch_unquantized_gemm().__name__ == "b200_unquantized_gemm"
    q = register_quant_configs()
    cfg_cls = get_quantization_config("fp8")
    assert cfg_cls is q["fp8"] and issubclass(cfg_cls, QuantizationConfig)
    cfg = cfg_cls.from_config({"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic",
                               "weight_block_size": [128, 128]})
    assert cfg.weight_block_size == [128, 128]
    with pytest.raises(ValueError):
        cfg_cls.from_config({"quant_method": "fp8", "weight_block_size": [64, 64]})


def test_weak_ref_tensor_is_a_dispatcher_op_when_the_extension_is_built():
    from vllm_kunlun_b200.ops import _ext
    if not _ext.available():
        pytest.skip("extension not built")
    assert hasattr(torch.ops._C_b200, "weak_ref_tensor") or hasattr(torch.ops._C, "weak_ref_tensor")


def test_gqa_builder_and_impl_run_on_upstreams_common_metadata():
    """Decode-first batch (two single-token decodes, then a 9-token and a 5-token prefill) through the builder and the
    implementation on CPU tensors (oracle path) against plain causal attention."""
    from types import SimpleNamespace

    from vllm.v1.attention.backend import CommonAttentionMetadata
    from vllm_kunlun_b200.attention.backends import GQABackend
    from vllm_kunlun_b200.ops.reference import attention as ra
    torch.manual_seed(0)
    H, Hkv, D, bs = 4, 2, 64, 16
    q_lens, ctx = [1, 1, 9, 5], [20, 3, 0, 7]
    seq = [c + q for q, c in zip(q_lens, ctx)]
    B, T = len(q_lens), sum(q_lens)
    nblk_per = [-(-s // bs) for s in seq]
    bt = torch.zeros(B, max(nblk_per), dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(nblk_per):
        bt[b, :n] = torch.arange(nxt, nxt + n)
        nxt += n
    cache = torch.zeros(GQABackend.get_kv_cache_shape(nxt, bs, Hkv, D))
    # history already in the cache
    hist_k, hist_v = {}, {}
    for b in range(B):
        hist_k[b], hist_v[b] = torch.randn(seq[b], Hkv, D), torch.randn(seq[b], Hkv, D)
        for p in range(ctx[b]):
            blk, off = int(bt[b, p // bs]), p % bs
            cache[blk, 0, :, off], cache[blk, 1, :, off] = hist_k[b][p], hist_v[b][p]
    qsl = torch.zeros(B + 1, dtype=torch.int32)
    qsl[1:] = torch.tensor(q_lens).cumsum(0)
    slots, keys, vals = [], [], []
    for b in range(B):
        for p in range(ctx[b], seq[b]):
            slots.append(int(bt[b, p // bs]) * bs + p % bs)
            keys.append(hist_k[b][p]); vals.append(hist_v[b][p])
    key, value = torch.stack(keys), torch.stack(vals)
    query = torch.randn(T, H, D)
    common = CommonAttentionMetadata(
        query_start_loc=qsl, query_start_loc_cpu=qsl, seq_lens=torch.tensor(seq, dtype=torch.int32), num_reqs=B,
        num_actual_tokens=T, max_query_len=max(q_lens), max_seq_len=max(seq), block_table_tensor=bt,
        slot_mapping=torch.tensor(slots, dtype=torch.int64), causal=True)
    spec = SimpleNamespace(block_size=bs, num_kv_heads=Hkv, head_size=D)
    vcfg = SimpleNamespace(
        model_config=SimpleNamespace(max_model_len=128, get_num_attention_heads=lambda par: H),
        speculative_config=None, parallel_config=SimpleNamespace(decode_context_parallel_size=1),
        scheduler_config=SimpleNamespace(max_num_seqs=8))
    builder = GQABackend.get_builder_cls()(spec, ["layers.0.attn"], vcfg, torch.device("cpu"))
    assert builder.reorder_batch_threshold == 1
    md = builder.build(0, common)
    assert (md.num_decodes, md.num_decode_tokens, md.num_prefills) == (2, 2, 2)
    impl = GQABackend.get_impl_cls()(H, D, D ** -0.5, Hkv, None, None, "auto", None)
    out = torch.full((T, H, D), float("nan"))
    impl.forward(None, query, key, value, cache, md, out)
    t = 0
    for b in range(B):
        ref = ra._attend(query[t:t + q_lens[b]], hist_k[b], hist_v[b], D ** -0.5, ctx[b], None, None)
        assert torch.allclose(out[t:t + q_lens[b]], ref.to(out.dtype), atol=1e-4, rtol=1e-4), b
        t += q_lens[b]
    # profiling call (no metadata) zero-fills
    assert impl.forward(None, query, key, value, cache, None, out).abs().sum() == 0


def test_upstream_c_namespace_ops_are_defined_with_upstream_schemas():
    """Upstream layers bind ``torch.ops._C.<op>`` in ``__init__``; the plugin defines them (its kernels on CUDA
    tensors, plain arithmetic otherwise) when upstream's own extension is not loaded."""
    from vllm_kunlun_b200.ops.oot_layers import define_upstream_c_ops
    define_upstream_c_ops()
    x = torch.randn(3, 8)
    out = torch.empty(3, 4)
    torch.ops._C.silu_and_mul(out, x)
    torch.testing.assert_close(out, torch.nn.functional.silu(x[:, :4]) * x[:, 4:])
    torch.ops._C.gelu_tanh_and_mul(out, x)
    torch.testing.assert_close(out, torch.nn.functional.gelu(x[:, :4], approximate="tanh") * x[:, 4:])
    r, w = torch.randn(3, 8), torch.rand(8) + 0.5
    x0, r0 = x.clone(), r.clone()
    torch.ops._C.fused_add_rms_norm(x, r, w, 1e-6)
    s = x0 + r0
    torch.testing.assert_close(r, s)
    torch.testing.assert_close(x, s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w)
    res = torch.empty_like(s)
    torch.ops._C.rms_norm(res, s, w, 1e-6)
    torch.testing.assert_close(res, x)


def test_glm47_tool_parser_is_an_upstream_tool_parser():
    """`--tool-call-parser glm47` resolves through upstream's manager to a `ToolParser` subclass with upstream's method
    signatures; complete and streaming extraction return upstream's protocol objects."""
    import inspect
    import json
    from types import SimpleNamespace

    from vllm.tool_parsers.abstract_tool_parser import ToolParser, ToolParserManager

    import vllm_kunlun_b200 as pkg
    pkg.register_tool_parser()
    cls = ToolParserManager.get_tool_parser("glm47")
    assert issubclass(cls, ToolParser)
    for name in ("extract_tool_calls", "extract_tool_calls_streaming"):
        assert list(inspect.signature(getattr(cls, name)).parameters) == \
            list(inspect.signature(getattr(ToolParser, name)).parameters)
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {
        "n": {"type": "integer"}, "s": {"type": "string"}}}}}]
    req = SimpleNamespace(tools=tools)
    tok = SimpleNamespace(get_vocab=lambda: {}, vocab={})
    text = "hi <tool_call>f\n<arg_key>n</arg_key><arg_value>4</arg_value><arg_key>s</arg_key><arg_value>x y</arg_value></tool_call>"
    p = cls(tok)
    info = p.extract_tool_calls(text, req)
    assert info.tools_called and info.content == "hi"
    assert info.tool_calls[0].function.name == "f" and json.loads(info.tool_calls[0].function.arguments) == {"n": 4, "s": "x y"}
    p = cls(tok)
    name, args, content, prev = None, "", "", ""
    for i in range(0, len(text), 5):
        piece = text[i:i + 5]
        d = p.extract_tool_calls_streaming(prev, prev + piece, piece, [], [], [], req)
        prev += piece
        if d is None:
            continue
        content += d.content or ""
        for tc in d.tool_calls:
            if tc.function.name:
                name = tc.function.name
            args += tc.function.arguments or ""
    assert name == "f" and content == "hi " and json.loads(args) == {"n": 4, "s": "x y"}
