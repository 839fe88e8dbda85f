"""Per-step attention metadata and the forward context.

One flat structure serves the GQA, MLA, sparse-MLA, indexer and GDN backends.  The reference keeps
separate classes with host *and* device copies of every length array because its kernels want both
(``KunlunMetadata`` ``v1/attention/backends/kunlun_attn.py:128-230``; ``MLACommonMetadata``
``mla/common.py:384-425``; ``FlashMLASparseMetadata`` ``mla/flashmla_sparse.py:152-182``;
``GDNAttentionMetadata`` ``gdn_attn.py:35-75``).  The CUDA kernels here read device tensors only;
the ``*_cpu`` mirrors exist for scheduling decisions and the CPU oracle path.

Batch order is decode-first (``kunlun_attn.py:509-546``): requests with ``q_len <= 1 + num_spec``
come first, prefills last.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class AttentionMetadata:
    num_tokens: int
    num_reqs: int
    positions: torch.Tensor  # [T] int64
    slot_mapping: torch.Tensor  # [T] int64, -1 = padding
    block_tables: torch.Tensor  # [B, max_blocks] int32
    seq_lens: torch.Tensor  # [B] int32 (context length after this step's tokens)
    query_start_loc: torch.Tensor  # [B+1] int32
    max_query_len: int
    max_seq_len: int
    num_decodes: int = 0
    num_decode_tokens: int = 0
    num_prefills: int = 0
    seq_lens_cpu: Optional[torch.Tensor] = None
    query_start_loc_cpu: Optional[torch.Tensor] = None
    req_id_per_token: Optional[torch.Tensor] = None  # [T] int32 (sparse MLA / indexer)
    # GDN / mamba-style state
    state_indices: Optional[torch.Tensor] = None  # [B] int32 slot in the state cache
    has_initial_state: Optional[torch.Tensor] = None  # [B] bool
    num_accepted_tokens: Optional[torch.Tensor] = None
    # speculative decoding
    num_spec_tokens: int = 0
    # logits are computed for these token rows only
    logits_indices: Optional[torch.Tensor] = None
    # scratch owned by the runner (split-KV partials etc.)
    workspace: Optional[Any] = None
    is_dummy: bool = False  # profile / warm-up run: attention impls may early-return
    extras: dict = field(default_factory=dict)

    @property
    def is_pure_decode(self) -> bool:
        return self.num_prefills == 0


@dataclass
class ForwardContext:
    attn: Optional[AttentionMetadata]
    kv_caches: list  # per layer: tensor or tuple of tensors
    pstate: Any
    capturing: bool = False
    lora: Optional[Any] = None
    extras: dict = field(default_factory=dict)


_CTX: Optional[ForwardContext] = None


def get_forward_context() -> ForwardContext:
    assert _CTX is not None, "forward context not set"
    return _CTX


@contextlib.contextmanager
def set_forward_context(ctx: ForwardContext):
    global _CTX
    prev = _CTX
    _CTX = ctx
    try:
        yield ctx
    finally:
        _CTX = prev
