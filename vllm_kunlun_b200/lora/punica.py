"""Punica wrapper: maps every token of the step to its adapter slot and applies shrink / expand.

Same surface as the reference's ``PunicaWrapperKunlun`` (``vllm_kunlun/lora/punica_wrapper/punica_kunlun.py``:
``add_shrink`` :273, ``add_expand`` :316, ``add_lora_linear`` :401, ``add_lora_logits`` :495, embedding :365),
which picks segment kernels (sgmv) for prefill and per-token kernels (bgmv) for decode.  Here both cases run
the same per-token kernels: the activation row is staged in shared memory once per token, so a segment
variant would not read fewer bytes, and a single code path keeps the step graph-capturable (the token ->
adapter vector lives at a fixed device address)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops


class PunicaWrapperB200:
    def __init__(self, max_num_batched_tokens: int, max_batches: int, device, **kwargs):
        self.device = torch.device(device)
        self.max_tokens = max_num_batched_tokens
        self.max_batches = max_batches
        self.token_lora_ids: Optional[torch.Tensor] = None  # [T] int32, -1 = no adapter
        self.sampler_lora_ids: Optional[torch.Tensor] = None  # [n_logit_rows] int32
        self.no_lora = True

    # ---- metadata
    def update_metadata(self, token_lora_ids: torch.Tensor, sampler_lora_ids: Optional[torch.Tensor] = None,
                        no_lora: bool = False):
        self.token_lora_ids = token_lora_ids
        self.sampler_lora_ids = sampler_lora_ids
        self.no_lora = no_lora

    @staticmethod
    def segments_to_token_ids(seq_lod: torch.Tensor, lora_ids: torch.Tensor) -> torch.Tensor:
        """Segment form (``seq_lod [S+1]``, ``lora_ids [S]``) -> per-token ids."""
        lens = (seq_lod[1:] - seq_lod[:-1]).long()
        return torch.repeat_interleave(lora_ids.int(), lens)

    # ---- primitives
    def add_shrink(self, x: torch.Tensor, lora_a_stacked: Sequence[torch.Tensor], scale: float = 1.0):
        """``[x @ A_i[id].T * scale for i in slices]`` as fp32 ``[T, r]`` buffers."""
        x2 = x.reshape(-1, x.shape[-1])
        return [ops.lora_shrink(x2, a, self.token_lora_ids[: x2.shape[0]], scale) for a in lora_a_stacked]

    def add_expand(self, y: torch.Tensor, h: Sequence[torch.Tensor], lora_b_stacked: Sequence[torch.Tensor],
                   output_slices: Sequence[int], offset_start: int = 0, add_inputs: bool = True):
        y2 = y.reshape(-1, y.shape[-1])
        off = offset_start
        for hi, b, n in zip(h, lora_b_stacked, output_slices):
            ops.lora_expand(hi, b, self.token_lora_ids[: y2.shape[0]], y2, off, add_inputs)
            off += n
        return y

    def add_lora_linear(self, y: torch.Tensor, x: torch.Tensor, lora_a_stacked, lora_b_stacked, scale: float,
                        output_slices: Sequence[int]):
        """``y[:, slice_i] += (x @ A_i.T * scale) @ B_i.T`` for every output slice of a (merged) linear."""
        if self.no_lora:
            return y
        h = self.add_shrink(x, lora_a_stacked, scale)
        return self.add_expand(y, h, lora_b_stacked, output_slices, 0, True)

    def add_lora_embedding(self, y: torch.Tensor, a_rows: torch.Tensor, lora_b_stacked: torch.Tensor):
        """Embedding LoRA: ``a_rows [T, r]`` (already gathered rows of A^T) expanded through B."""
        if self.no_lora:
            return y
        ops.lora_expand(a_rows.float(), lora_b_stacked, self.token_lora_ids[: y.shape[0]], y, 0, True)
        return y

    def add_lora_logits(self, y: torch.Tensor, x: torch.Tensor, lora_a_stacked: torch.Tensor,
                        lora_b_stacked: torch.Tensor, scale: float = 1.0):
        if self.no_lora:
            return y
        ids = self.sampler_lora_ids[: x.shape[0]]
        h = ops.lora_shrink(x, lora_a_stacked, ids, scale)
        ops.lora_expand(h, lora_b_stacked, ids, y, 0, True)
        return y
