"""Out-of-tree layer implementations registered with upstream vLLM's ``CustomOp`` / ``PluggableLayer`` registries.

Reference: the seven ``@CustomOp.register_oot`` sites of the plugin plus its pluggable router
(``ops/layernorm.py:51,108``, ``ops/rotary_embedding/kunlun_rope.py:31``, ``kunlun_mrope.py:32``,
``kunlun_deepseek_rope.py:32``, ``ops/vocab_parallel_embedding.py:75``, ``ops/fused_moe/layer.py:16``,
``ops/fused_moe/router/gate_linear.py:10``) and the replaced unquantised linear method (``ops/linear.py:49-72``).
On this platform ``CustomOp.dispatch_forward`` picks ``forward_oot``; each ``forward_oot`` below runs this
package's sm_100a kernel for CUDA tensors and falls back to upstream's ``forward_native`` for anything the kernel
does not serve (fp32 activations, partial rotary dims the kernel does not know, ...).

``register_oot_layers()`` is idempotent and a no-op when vLLM is not importable.
"""
from __future__ import annotations

import torch

from .. import ops

_DONE = [False]
REGISTERED: dict = {}


def _kernel_dtype(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)


def register_oot_layers() -> dict:
    if _DONE[0]:
        return REGISTERED
    try:
        from vllm.model_executor.custom_op import CustomOp, op_registry_oot
        from vllm.model_executor.layers.activation import SiluAndMul
        from vllm.model_executor.layers.layernorm import GemmaRMSNorm, RMSNorm
        from vllm.model_executor.layers.rotary_embedding import RotaryEmbedding
        from vllm.model_executor.layers.vocab_parallel_embedding import VocabParallelEmbedding
    except Exception:  # vLLM absent: nothing to register
        return REGISTERED
    _DONE[0] = True

    def reg(base, name):
        def deco(cls):
            if name not in op_registry_oot:
                base.register_oot(name=name)(cls)
            REGISTERED[name] = cls
            return cls
        return deco

    @reg(RMSNorm, "RMSNorm")
    class B200RMSNorm(RMSNorm):
        """``residual += x; x = rmsnorm(residual) * w`` in place, one kernel (``_C::add_rmsnorm`` / ``_C::rmsnorm``)."""

        def forward_oot(self, x, residual=None):
            if not _kernel_dtype(x) or self.variance_size_override is not None or not self.has_weight:
                return self.forward_native(x, residual)
            w = self.weight.data
            if w.dtype != x.dtype:
                w = w.to(x.dtype)
            shape = x.shape
            x2 = x.reshape(-1, shape[-1])
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            if residual is None:
                return ops.rmsnorm(x2, w, self.variance_epsilon).reshape(shape)
            r2 = residual.reshape(-1, shape[-1])
            if not r2.is_contiguous():
                return self.forward_native(x, residual)
            ops.add_rmsnorm(x2, r2, w, self.variance_epsilon)  # in place on both, like upstream's fused op
            return x2.reshape(shape), residual

    @reg(GemmaRMSNorm, "GemmaRMSNorm")
    class B200GemmaRMSNorm(GemmaRMSNorm):
        """The ``(1 + w)`` variant (``_C::gemma_rmsnorm`` / ``_C::gemma_add_rmsnorm``)."""

        def forward_oot(self, x, residual=None):
            if not _kernel_dtype(x):
                return self.forward_native(x, residual)
            w = self.weight.data.to(x.dtype)
            shape = x.shape
            x2 = x.reshape(-1, shape[-1]).contiguous()
            if residual is None:
                return ops.rmsnorm(x2, w, self.variance_epsilon, True).reshape(shape)
            r2 = residual.reshape(-1, shape[-1])
            if not r2.is_contiguous():
                return self.forward_native(x, residual)
            ops.add_rmsnorm(x2, r2, w, self.variance_epsilon, True)
            return x2.reshape(shape), residual

    @reg(SiluAndMul, "SiluAndMul")
    class B200SiluAndMul(SiluAndMul):
        def forward_oot(self, x):
            if not _kernel_dtype(x) or not x.is_contiguous():
                return self.forward_native(x)
            return ops.silu_and_mul(x)

    @reg(RotaryEmbedding, "RotaryEmbedding")
    class B200RotaryEmbedding(RotaryEmbedding):
        """In-place neox / gpt-j rotary on ``q`` and ``k`` from an fp32 copy of upstream's cos/sin cache."""

        def forward_oot(self, positions, query, key=None):
            if (not _kernel_dtype(query) or key is None or self.rotary_dim != self.head_size
                    or not query.is_contiguous() or not key.is_contiguous()):
                return self.forward_native(positions, query, key)
            cache = getattr(self, "_b200_cos_sin", None)
            if cache is None or cache.device != query.device:
                cache = self._b200_cos_sin = self.cos_sin_cache.to(device=query.device, dtype=torch.float32).contiguous()
            T = positions.numel()
            q2, k2 = query.view(T, -1), key.view(T, -1)
            ops.rope(q2, k2, positions.reshape(-1).long(), cache, self.head_size, self.is_neox_style)
            return query, key

    @reg(VocabParallelEmbedding, "VocabParallelEmbedding")
    class B200VocabParallelEmbedding(VocabParallelEmbedding):
        """Masked gather in one kernel (rows outside the shard give zeros), then the TP all-reduce (call site C4)."""

        def forward(self, input_):
            w = getattr(self, "weight", None)
            if (w is None or not w.is_cuda or w.dtype not in (torch.bfloat16, torch.float16)
                    or self.shard_indices.num_added_elements > 0
                    or type(self.quant_method).__name__ != "UnquantizedEmbeddingMethod"):
                return super().forward(input_)
            from vllm.distributed import tensor_model_parallel_all_reduce
            out = ops.embedding(input_.reshape(-1).long(), w[: self.shard_indices.num_org_elements],
                                self.shard_indices.org_vocab_start_index)
            out = out.reshape(*input_.shape, w.shape[1])
            return tensor_model_parallel_all_reduce(out) if self.tp_size > 1 else out

    _patch_unquantized_gemm()
    define_upstream_c_ops()
    return REGISTERED


_C_LIB: list = []


def define_upstream_c_ops() -> list:
    """Give ``torch.ops._C`` the element-wise ops that upstream's layers bind at construction time
    (``SiluAndMul.__init__`` reads ``torch.ops._C.silu_and_mul`` on every CUDA-like platform, whatever
    ``forward_*`` is dispatched later), with upstream's schemas and this package's kernels behind them.  Upstream's
    own ``vllm._C`` is not loaded under this platform (``B200Platform.import_kernels``), so the names are free; a
    name that IS already defined is left alone.  The reference fills the same namespace with its device's kernels
    (``vllm_kunlun/ops/_kunlun_ops.py``, ``vllm_kunlun/vllm_utils_wrapper.py``).  Returns the names defined here."""
    if _C_LIB:
        return _C_LIB[1]
    lib = torch.library.Library("_C", "FRAGMENT")
    done: list = []

    def has(name):
        try:
            getattr(torch.ops._C, name)
            return True
        except (AttributeError, RuntimeError):
            return False

    def define(name, schema, fn):
        if has(name):
            return
        lib.define(f"{name}{schema}")
        lib.impl(name, fn, "CompositeExplicitAutograd")
        done.append(name)

    def gated(act):
        def fn(out, x):
            if act != "gelu" and _kernel_dtype(x) and x.is_contiguous():  # erf-GELU has no kernel here
                out.copy_(ops.act_and_mul(x, act))
            else:
                d = x.shape[-1] // 2
                g = {"silu": torch.nn.functional.silu,
                     "gelu": torch.nn.functional.gelu,
                     "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[act]
                out.copy_(g(x[..., :d]) * x[..., d:])
        return fn

    def mul_and_silu(out, x):
        d = x.shape[-1] // 2
        out.copy_(x[..., :d] * torch.nn.functional.silu(x[..., d:]))

    def fatrelu_and_mul(out, x, threshold=0.0):
        d = x.shape[-1] // 2
        out.copy_(torch.nn.functional.threshold(x[..., :d], threshold, 0.0) * x[..., d:])

    def swigluoai_and_mul(out, x, alpha=1.702, limit=7.0):
        g, u = x[..., ::2].clamp(max=limit), x[..., 1::2].clamp(-limit, limit)
        out.copy_((u + 1) * g * torch.sigmoid(g * alpha))

    def unary(f):
        def fn(out, x):
            out.copy_(f(x))
        return fn

    def gelu_new(x):
        return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x.pow(3))))

    def gelu_fast(x):
        return 0.5 * x * (1.0 + torch.tanh(x * 0.7978845608 * (1.0 + 0.044715 * x * x)))

    def gelu_quick(x):
        return ops.quick_gelu(x) if _kernel_dtype(x) and x.is_contiguous() else x * torch.sigmoid(1.702 * x)

    def rms_norm(result, x, weight, epsilon):
        x2 = x.reshape(-1, x.shape[-1])
        if _kernel_dtype(x) and x2.is_contiguous():
            result.copy_(ops.rmsnorm(x2, weight.to(x.dtype), epsilon).view_as(result))
        else:
            v = x.float()
            result.copy_((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + epsilon) * weight.float()).to(x.dtype))

    def fused_add_rms_norm(x, residual, weight, epsilon):
        x2, r2 = x.view(-1, x.shape[-1]), residual.view(-1, x.shape[-1])
        if _kernel_dtype(x) and x2.is_contiguous() and r2.is_contiguous():
            ops.add_rmsnorm(x2, r2, weight.to(x.dtype), epsilon)
        else:
            v = x.float() + residual.float()
            residual.copy_(v.to(x.dtype))
            v = residual.float()
            x.copy_((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + epsilon) * weight.float()).to(x.dtype))

    def rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox):
        T = positions.numel()
        rot = cos_sin_cache.shape[-1]
        assert rot == head_size and key is not None and _kernel_dtype(query), \
            "_C::rotary_embedding on this platform: full rotary dim, 16-bit q and k"
        ops.rope(query.view(T, -1), key.view(T, -1), positions.reshape(-1).long(),
                 cos_sin_cache.to(torch.float32), head_size, is_neox)

    for name, act in (("silu_and_mul", "silu"), ("gelu_and_mul", "gelu"), ("gelu_tanh_and_mul", "gelu_tanh")):
        define(name, "(Tensor! out, Tensor input) -> ()", gated(act))
    define("mul_and_silu", "(Tensor! out, Tensor input) -> ()", mul_and_silu)
    define("fatrelu_and_mul", "(Tensor! out, Tensor input, float threshold) -> ()", fatrelu_and_mul)
    define("swigluoai_and_mul", "(Tensor! out, Tensor input, float alpha=1.702, float limit=7.0) -> ()",
           swigluoai_and_mul)
    define("gelu_new", "(Tensor! out, Tensor input) -> ()", unary(gelu_new))
    define("gelu_fast", "(Tensor! out, Tensor input) -> ()", unary(gelu_fast))
    define("gelu_quick", "(Tensor! out, Tensor input) -> ()", unary(gelu_quick))
    define("rms_norm", "(Tensor! result, Tensor input, Tensor weight, float epsilon) -> ()", rms_norm)
    define("fused_add_rms_norm", "(Tensor! input, Tensor! residual, Tensor weight, float epsilon) -> ()",
           fused_add_rms_norm)
    define("rotary_embedding", "(Tensor positions, Tensor! query, Tensor!? key, int head_size, Tensor cos_sin_cache, "
           "bool is_neox) -> ()", rotary_embedding)
    _C_LIB.extend([lib, done])
    return done


def b200_unquantized_gemm(layer, x: torch.Tensor, weight: torch.Tensor, bias=None) -> torch.Tensor:
    """``y = x @ W.T (+ b)`` for upstream's ``UnquantizedLinearMethod`` on the tcgen05 GEMM (no library GEMM);
    shapes or dtypes the kernel does not take go to ``F.linear``."""
    if (_kernel_dtype(x) and weight.is_cuda and weight.dtype == x.dtype and weight.dim() == 2 and weight.is_contiguous()
            and weight.shape[1] % 8 == 0 and x.shape[-1] == weight.shape[1]
            and (bias is None or (bias.dtype == x.dtype and bias.is_contiguous()))):
        return ops.linear(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


def _patch_unquantized_gemm() -> None:
    """Upstream picks the unquantised GEMM by platform kind with no out-of-tree hook
    (``vllm/model_executor/layers/utils.py::dispatch_unquantized_gemm``); the reference replaces the linear method
    outright (``ops/linear.py:71-72``).  Here only the dispatch function is replaced."""
    try:
        from vllm.model_executor.layers import utils as U
    except Exception:
        return
    if getattr(U.dispatch_unquantized_gemm, "_b200", False):
        return

    def dispatch_unquantized_gemm():
        return b200_unquantized_gemm
    dispatch_unquantized_gemm._b200 = True
    U.dispatch_unquantized_gemm = dispatch_unquantized_gemm
    try:  # modules that imported the symbol by name
        from vllm.model_executor.layers import linear as L
        if hasattr(L, "dispatch_unquantized_gemm"):
            L.dispatch_unquantized_gemm = dispatch_unquantized_gemm
    except Exception:
        pass
