"""``PunicaWrapperB200`` for upstream vLLM's LoRA layers: a ``PunicaWrapperBase`` subclass with upstream's method
signatures on this package's per-token shrink / expand kernels.

Reference: ``PunicaWrapperKunlun`` (``vllm_kunlun/lora/punica_wrapper/punica_kunlun.py``: ``add_shrink`` :273,
``add_expand`` :316, ``add_lora_embedding`` :365, ``add_lora_linear`` :401, ``add_lora_logits`` :495), selected by
``Platform.get_punica_wrapper`` (``platforms/kunlun.py:342-347``).  The reference picks segment kernels (sgmv) for
prefill and per-token kernels (bgmv) for decode; here one per-token path serves both (the activation row is staged
in shared memory once per token, so a segment variant would not read fewer bytes).

Upstream stacks adapter weights as ``lora_a [max_loras, 1, rank, in]`` and ``lora_b [max_loras, 1, out, rank]``;
the kernels take ``[max_loras, rank, in]`` / ``[max_loras, out, rank]`` views of the same memory.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .. import ops

try:
    from vllm.lora.punica_wrapper.punica_base import PunicaWrapperBase
except Exception:  # pragma: no cover
    PunicaWrapperBase = object  # type: ignore


def _w3(w: torch.Tensor) -> torch.Tensor:
    return w.squeeze(1) if w.dim() == 4 else w


class PunicaWrapperB200(PunicaWrapperBase):
    def __init__(self, max_num_batched_tokens: int, max_batches: int, device: Union[torch.device, str], **kwargs):
        super().__init__(max_num_batched_tokens, max_batches, device, **kwargs)

    def _ids(self, n: int) -> torch.Tensor:
        return self.token_lora_indices[:n].int()

    def add_shrink(self, y, x: torch.Tensor, lora_a_stacked, scale: float, **kwargs):
        """``y[i] += (x @ lora_a_stacked[i]) * scale`` for every slice ``i``."""
        x2 = x.reshape(-1, x.shape[-1])
        for i, a in enumerate(lora_a_stacked):
            h = ops.lora_shrink(x2, _w3(a), self._ids(x2.shape[0]), scale)
            y[i].add_(h.to(y[i].dtype))
        return y

    def add_expand(self, y: torch.Tensor, x, lora_b_stacked, output_slices, offset_start: int = 0,
                   add_inputs: bool = True, **kwargs):
        y2 = y.reshape(-1, y.shape[-1])
        off = offset_start
        for i, (b, n) in enumerate(zip(lora_b_stacked, output_slices)):
            ops.lora_expand(x[i].float(), _w3(b), self._ids(y2.shape[0]), y2, off, add_inputs)
            off += n
        return y

    def add_lora_embedding(self, y: torch.Tensor, x: torch.Tensor, lora_b_stacked: torch.Tensor,
                           add_inputs: bool = True, **kwargs):
        ops.lora_expand(x.float(), _w3(lora_b_stacked), self._ids(y.shape[0]), y, 0, add_inputs)
        return y

    def add_lora_linear(self, y: torch.Tensor, x: torch.Tensor, lora_a_stacked, lora_b_stacked, scale: float,
                        output_slices, *, buffer: Optional[tuple] = None, **kwargs):
        """``y[:, slice_i] += (x @ A_i^T * scale) @ B_i^T``; the rank-sized intermediates stay in fp32."""
        if self.no_lora:
            return y
        x2 = x.reshape(-1, x.shape[-1])
        y2 = y.reshape(-1, y.shape[-1])
        ids = self._ids(x2.shape[0])
        off = 0
        for a, b, n in zip(lora_a_stacked, lora_b_stacked, output_slices):
            h = ops.lora_shrink(x2, _w3(a), ids, scale)
            ops.lora_expand(h, _w3(b), ids, y2, off, True)
            off += n
        return y

    def add_lora_logits(self, y: torch.Tensor, x: torch.Tensor, lora_a_stacked: torch.Tensor,
                        lora_b_stacked: torch.Tensor, scale, *, buffer: Optional[torch.Tensor] = None, **kwargs):
        if self.no_lora:
            return y
        y2 = y.reshape(-1, y.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        ids = self.sampler_indices[: x2.shape[0]].int()
        h = ops.lora_shrink(x2, _w3(lora_a_stacked), ids, scale)
        ops.lora_expand(h, _w3(lora_b_stacked), ids, y2, 0, True)
        return y
