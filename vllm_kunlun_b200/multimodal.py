"""Image inputs of the serving front end: OpenAI ``image_url`` content parts -> the tensors the Qwen-VL towers take.

The reference serves its vision-language models through upstream's chat endpoint, whose processor resizes every image
to a multiple of ``patch_size * merge_size`` inside a pixel budget, normalises it and cuts it into flattened patches
ordered merge-block by merge-block (``vllm_kunlun/models/qwen2_vl.py:1012-1118`` and ``qwen2_5_vl.py`` consume that
layout).  This module does the same work without a processor object:

* :func:`load_image` - a ``data:`` URI, a ``file://`` URL or a local path -> RGB ``PIL.Image``;
* :func:`smart_resize` - the target height / width;
* :class:`QwenImagePreprocessor` - images -> ``pixel_values [sum(t*h*w), C * temporal_patch * patch * patch]`` and
  ``image_grid_thw``;
* :class:`InternImagePreprocessor` - InternVL's tile grid + thumbnail;
* :func:`expand_placeholders` - a chat template writes ONE placeholder token per image; the engine wants one per
  merged patch;
* :func:`collect_images` - the ``image_url`` / ``image`` parts of an OpenAI ``messages`` list, in order.
"""
from __future__ import annotations

import base64
import io
import math
import os
from typing import Optional, Sequence

import torch

# CLIP statistics: the defaults of the Qwen2-VL / Qwen2.5-VL processors (Qwen3-VL uses 0.5 / 0.5)
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def load_image(url: str):
    """``data:image/...;base64,....``, ``file:///path`` or a path -> RGB ``PIL.Image``.  Remote URLs are refused:
    a serving node fetches nothing on a client's behalf unless the operator enables it (``B200_ALLOW_REMOTE_IMAGES``)."""
    from PIL import Image
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("a data: URI of an image must be base64-encoded")
        raw = base64.b64decode(payload, validate=False)
        return Image.open(io.BytesIO(raw)).convert("RGB")
    if url.startswith("http://") or url.startswith("https://"):
        from . import envs
        if not envs.B200_ALLOW_REMOTE_IMAGES:
            raise ValueError("remote image URLs are not fetched; send the image as a data: URI")
        import urllib.request
        with urllib.request.urlopen(url, timeout=10) as r:
            return Image.open(io.BytesIO(r.read(64 << 20))).convert("RGB")
    path = url[len("file://"):] if url.startswith("file://") else url
    if not os.path.isfile(path):
        raise ValueError(f"no such image file: {path}")
    return Image.open(path).convert("RGB")


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Height and width, both multiples of ``factor``, closest to the input with ``min_pixels <= h * w <=
    max_pixels`` and the aspect ratio kept as far as the rounding allows."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError(f"the aspect ratio of a {height} x {width} image is beyond 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


class QwenImagePreprocessor:
    """Resize (bicubic), scale to [0, 1], normalise, repeat the frame ``temporal_patch`` times and flatten into
    patches in the towers' order: for every block of ``merge x merge`` patches, row-major over blocks, the patches of
    the block, each as (channel, frame, y, x)."""

    def __init__(self, patch: int = 14, temporal_patch: int = 2, merge: int = 2, min_pixels: int = 56 * 56,
                 max_pixels: int = 28 * 28 * 1280, mean: Sequence[float] = CLIP_MEAN, std: Sequence[float] = CLIP_STD):
        self.patch, self.temporal_patch, self.merge = patch, temporal_patch, merge
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(mean, dtype=torch.float32).view(3, 1, 1)
        self.std = torch.tensor(std, dtype=torch.float32).view(3, 1, 1)

    @classmethod
    def from_config(cls, vision: dict, processor: Optional[dict] = None):
        """``vision``: the model configuration's vision dictionary; ``processor``: the checkpoint's
        ``preprocessor_config.json`` when there is one (pixel budget, statistics)."""
        p = processor or {}
        size = p.get("size") or {}
        kw = dict(patch=vision["patch"], temporal_patch=vision["temporal_patch"], merge=vision["merge"])
        factor = kw["patch"] * kw["merge"]
        kw["min_pixels"] = int(p.get("min_pixels") or size.get("shortest_edge") or 4 * factor * factor)
        kw["max_pixels"] = int(p.get("max_pixels") or size.get("longest_edge") or 1280 * factor * factor)
        if p.get("image_mean"):
            kw["mean"], kw["std"] = p["image_mean"], p["image_std"]
        elif vision.get("patch_bias"):      # Qwen3-VL
            kw["mean"], kw["std"] = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)
        return cls(**kw)

    def one(self, image) -> tuple[torch.Tensor, tuple[int, int, int]]:
        from PIL import Image
        import numpy as np
        W, H = image.size
        h, w = smart_resize(H, W, self.patch * self.merge, self.min_pixels, self.max_pixels)
        arr = np.asarray(image.resize((w, h), resample=Image.Resampling.BICUBIC), dtype=np.uint8)
        x = (torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0 - self.mean) / self.std   # [3, h, w]
        p, m, tp = self.patch, self.merge, self.temporal_patch
        gh, gw = h // p, w // p
        x = x.unsqueeze(0).expand(tp, -1, -1, -1)                                                     # frames
        x = x.reshape(tp, 3, gh // m, m, p, gw // m, m, p)
        # -> (block row, block col, row in block, col in block, channel, frame, y, x)
        x = x.permute(2, 5, 3, 6, 1, 0, 4, 7).reshape(gh * gw, 3 * tp * p * p)
        return x.contiguous(), (1, gh, gw)

    def __call__(self, images) -> tuple[torch.Tensor, list]:
        outs = [self.one(im) for im in images]
        return torch.cat([o[0] for o in outs]), [list(o[1]) for o in outs]

    def tokens_per_image(self, grid) -> int:
        t, h, w = grid
        return t * h * w // (self.merge * self.merge)

    def mm_data(self, pixel_values, grids) -> dict:
        return {"pixel_values": pixel_values, "image_grid_thw": grids}


IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


class InternImagePreprocessor:
    """InternVL's tiling: the image is resized to the grid of ``image_size`` tiles (at most ``max_tiles``) whose
    aspect ratio is closest to its own, cut into tiles, and - when there is more than one tile - a thumbnail of the
    whole image is appended; every tile is normalised with the ImageNet statistics and flattened into patches
    ``[tiles, (image_size / patch)^2, 3 * patch * patch]`` (row-major patches, each as (channel, y, x)).  One tile
    becomes ``(image_size / patch * downsample)^2`` placeholder tokens."""

    def __init__(self, image_size: int = 448, patch: int = 14, downsample: float = 0.5, min_tiles: int = 1,
                 max_tiles: int = 12, use_thumbnail: bool = True):
        self.image_size, self.patch, self.downsample = image_size, patch, downsample
        self.min_tiles, self.max_tiles, self.use_thumbnail = min_tiles, max_tiles, use_thumbnail
        self.mean = torch.tensor(IMAGENET_MEAN, dtype=torch.float32).view(3, 1, 1)
        self.std = torch.tensor(IMAGENET_STD, dtype=torch.float32).view(3, 1, 1)
        self.tokens_per_tile = int(image_size // patch * downsample) ** 2

    @classmethod
    def from_config(cls, vision: dict, processor: Optional[dict] = None):
        p = processor or {}
        return cls(image_size=vision.get("image_size", 448), patch=vision["patch"], downsample=vision.get("downsample", 0.5),
                   min_tiles=int(p.get("min_dynamic_patch", p.get("min_patches", 1))),
                   max_tiles=int(p.get("max_dynamic_patch", p.get("max_patches", 12))),
                   use_thumbnail=bool(p.get("use_thumbnail", True)))

    def tile_grid(self, width: int, height: int) -> tuple[int, int]:
        """(columns, rows) of the tile grid: the admissible ratio closest to the image's; on a tie the larger grid
        wins when the image has more than half of that grid's pixels."""
        ratios = sorted({(i, j) for n in range(self.min_tiles, self.max_tiles + 1) for i in range(1, n + 1)
                         for j in range(1, n + 1) if self.min_tiles <= i * j <= self.max_tiles}, key=lambda r: r[0] * r[1])
        aspect, best, best_diff = width / height, (1, 1), float("inf")
        for i, j in ratios:
            diff = abs(aspect - i / j)
            if diff < best_diff:
                best, best_diff = (i, j), diff
            elif diff == best_diff and width * height > 0.5 * self.image_size ** 2 * i * j:
                best = (i, j)
        return best

    def _tile(self, image) -> torch.Tensor:
        import numpy as np
        arr = np.asarray(image, dtype=np.uint8)
        x = (torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0 - self.mean) / self.std
        g, p = self.image_size // self.patch, self.patch
        return x.view(3, g, p, g, p).permute(1, 3, 0, 2, 4).reshape(g * g, 3 * p * p)

    def one(self, image) -> torch.Tensor:
        from PIL import Image
        W, H = image.size
        cols, rows = self.tile_grid(W, H)
        s = self.image_size
        big = image.resize((s * cols, s * rows), resample=Image.Resampling.BICUBIC)
        tiles = [big.crop((c * s, r * s, (c + 1) * s, (r + 1) * s)) for r in range(rows) for c in range(cols)]
        if self.use_thumbnail and len(tiles) > 1:
            tiles.append(image.resize((s, s), resample=Image.Resampling.BICUBIC))
        return torch.stack([self._tile(t) for t in tiles])

    def __call__(self, images) -> tuple[torch.Tensor, list]:
        """-> (``[sum(tiles), patches, patch_dim]``, tiles per image)."""
        outs = [self.one(im) for im in images]
        return torch.cat(outs), [int(o.shape[0]) for o in outs]

    def tokens_per_image(self, tiles: int) -> int:
        return tiles * self.tokens_per_tile

    def mm_data(self, pixel_values, tiles) -> dict:
        return {"pixel_values": pixel_values}


def expand_placeholders(token_ids: Sequence[int], token_id: int, counts: Sequence[int]) -> list:
    """Every run of ``token_id`` stands for one image: replace the k-th run by ``counts[k]`` copies."""
    out, k, i, n = [], 0, 0, len(token_ids)
    while i < n:
        if token_ids[i] != token_id:
            out.append(token_ids[i])
            i += 1
            continue
        while i < n and token_ids[i] == token_id:
            i += 1
        if k >= len(counts):
            raise ValueError(f"the prompt has more image placeholders than the request has images ({len(counts)})")
        out += [token_id] * counts[k]
        k += 1
    if k != len(counts):
        raise ValueError(f"{len(counts)} images but {k} image placeholders in the prompt")
    return out


def collect_images(messages) -> list:
    """URLs of the image parts of an OpenAI ``messages`` list, in prompt order."""
    urls = []
    for m in messages or ():
        c = m.get("content")
        if not isinstance(c, list):
            continue
        for part in c:
            if not isinstance(part, dict):
                continue
            if part.get("type") == "image_url" or "image_url" in part:
                u = part.get("image_url")
                urls.append(u.get("url") if isinstance(u, dict) else u)
            elif part.get("type") == "image" and isinstance(part.get("image"), str):
                urls.append(part["image"])
    return urls
