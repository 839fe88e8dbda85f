"""CUDA entries for quantised linears: dynamic 1x128 fp8 activation quantisation feeding the
block-scaled tcgen05 GEMM (``csrc/gemm/gemm_grouped.cu``), and int8 W8A8."""
from __future__ import annotations

import torch

import os

from . import _ext

# decode-sized fp8 linears on the cluster split-K kernel (csrc/gemm/gemm_decode.cu); B200_DECODE_FP8=0 keeps them on
# the grouped kernel
DECODE_FP8 = [os.environ.get("B200_DECODE_FP8", "1") != "0"]


def quant_fp8_group_cuda(x: torch.Tensor, group: int = 128, ue8m0: bool = False, transposed: bool = False):
    """``(q, scale)``; ``scale`` is ``[rows, K/128]`` (or the kernel's transposed ``[K/128, stride]``)."""
    assert group == 128
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    q, st = _ext.C().quant_fp8_group(x2, ue8m0, None, 4)
    q = q.view(torch.float8_e4m3fn)
    if transposed:
        return q, st
    return q.reshape(*lead, -1), st[:, : x2.shape[0]].T.reshape(*lead, -1)


def fp8_linear_cuda(x, w_fp8, w_scale_inv, bias=None, block=(128, 128), out_dtype=torch.bfloat16):
    assert tuple(block) == (128, 128), "the fp8 GEMM is specialised for 128x128 weight blocks"
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    C = _ext.C()
    q, st = C.quant_fp8_group(x2, False, None, 4)
    N = w_fp8.shape[0]
    out = torch.empty(x2.shape[0], N, dtype=out_dtype, device=x.device)
    if (DECODE_FP8[0] and x2.shape[0] <= 32 and w_scale_inv.dim() == 2 and x2.shape[1] % 128 == 0
            and out_dtype in (torch.bfloat16, torch.float16)):
        # decode-sized call: cluster split-K kernel (every SM streams weight bytes; reduction in shared memory)
        C.gemm_decode_fp8(out, q, w_fp8.view(torch.uint8), bias, st, w_scale_inv.contiguous(), 0)
        return out.reshape(*lead, N)
    ws = w_scale_inv if w_scale_inv.dim() == 3 else w_scale_inv.unsqueeze(0)
    C.grouped_gemm(out, q, w_fp8.view(torch.uint8), None, bias, st, ws.contiguous(), 0)
    return out.reshape(*lead, N)


# W8A8 on the int8 tensor-core path (kind::i8); B200_INT8_TC=0 de-quantises the weight once and runs the 16-bit GEMM
INT8_TC = [os.environ.get("B200_INT8_TC", "1") != "0"]


def int8_linear_cuda(x2, w_q, w_scale, bias, input_scale, out_dtype):
    """W8A8 int8 (``quantization/kernels/scale_mm.py:43-90`` of the reference): activations are quantised per
    token (dynamic) or with the checkpoint's per-tensor scale (static) by ``quant_int8_token_kernel``, the product
    runs on ``tcgen05.mma.kind::i8`` with s32 accumulators, and the epilogue applies ``a_scale[t] * w_scale[n]``."""
    K = x2.shape[1]
    if (INT8_TC[0] and out_dtype in (torch.bfloat16, torch.float16) and K % 16 == 0 and w_q.dtype == torch.int8
            and w_q.is_contiguous() and x2.dtype in (torch.bfloat16, torch.float16, torch.float32)):
        C = _ext.C()
        xin = x2 if x2.stride(1) == 1 else x2.contiguous()
        st = None if input_scale is None else input_scale.float().reshape(-1).contiguous()
        q, s = C.quant_int8_token(xin, st)
        out = torch.empty(x2.shape[0], w_q.shape[0], dtype=out_dtype, device=x2.device)
        ws = w_scale.float().reshape(-1).contiguous()
        b = None if bias is None else bias.to(out_dtype)
        C.gemm_int8(out, q, w_q, b, s, ws)
        return out
    from .gemm_cuda import gemm_bf16
    key = "_b200_dequant"
    wd = getattr(w_q, key, None)
    if wd is None:
        wd = (w_q.float() * w_scale.float().reshape(-1, 1)).to(out_dtype)
        setattr(w_q, key, wd)
    return gemm_bf16(x2.to(out_dtype), wd, bias)
