"""Checkpoint I/O: Hugging Face safetensors directories (single file or sharded with an index).

Inference-only, so "checkpoint / resume" is weight loading: iterate ``(name, tensor)`` pairs and let
the model's ``load_weights`` map them onto fused / sharded parameters - the flow of the reference
(``models/deepseek_v2.py:1285-1413``; per-parameter sharding in ``ops/linear.py:137-424``).  fp8 checkpoints
carry ``*.weight_scale_inv`` tensors that travel through the same path."""
from __future__ import annotations

import glob
import json
import os
from typing import Iterator

import torch


def load_safetensors(path: str, device: str = "cpu") -> Iterator[tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(os.path.basename(p) for p in glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for fn in files:
        with safe_open(os.path.join(path, fn), framework="pt", device=device) as f:
            for name in f.keys():
                yield name, f.get_tensor(name)


def save_safetensors(state: dict, path: str, config: dict | None = None, max_shard_bytes: int = 2 << 30) -> None:
    """Write an HF-style directory (used by tests and by tools that export random-init checkpoints)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    shards, cur, size = [], {}, 0
    for k, v in state.items():
        nbytes = v.numel() * v.element_size()
        if cur and size + nbytes > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v.contiguous()
        size += nbytes
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn))
        weight_map.update({k: fn for k in sh})
    if len(shards) > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": weight_map}, f)
    if config is not None:
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(config, f)
