"""Image decoding, resizing and per-architecture preprocessing.

Parity: Gemma3/ImageProcessor.cs (decode to RGBA, alpha composited on white, bilinear resize with
half-pixel centres and no anti-aliasing :414-466, mean / std 0.5, fixed 896 x 896, 256 tokens per
image, token ids :24-27), Gemma4ImageProcessor.cs (align to patch * merge = 48, at most 280 output
tokens), Qwen35/ImageProcessor.cs (SmartResize to multiples of patch * merge within a pixel
budget :38-60), Mistral3ImageProcessor.cs (longest edge 1540, CLIP mean / std, patch-aligned
:39-66).  Decoding uses Pillow (PNG, JPEG, and HEIC when a HEIF plug-in is installed).
"""
from __future__ import annotations

import math
from typing import Tuple

import numpy as np
import torch


def decode_image_rgba(path: str) -> torch.Tensor:
    """uint8 ``[H, W, 4]``."""
    from PIL import Image
    try:
        with Image.open(path) as im:
            return torch.from_numpy(np.array(im.convert("RGBA"), dtype=np.uint8))
    except Exception as e:
        raise ValueError(f"Only PNG, JPEG, and HEIC/HEIF image formats are supported ({path}: {e})") from e


def read_image_dimensions(path: str) -> Tuple[int, int]:
    """(width, height) without decoding the pixels."""
    from PIL import Image
    with Image.open(path) as im:
        return im.size


def composite_over_white(rgba: torch.Tensor) -> torch.Tensor:
    """float32 ``[H, W, 3]`` in 0..255."""
    a = rgba[..., 3:4].float() / 255.0
    return rgba[..., :3].float() * a + 255.0 * (1.0 - a)


def resize_bilinear_chw(rgb: torch.Tensor, dst_w: int, dst_h: int) -> torch.Tensor:
    """``rgb`` float ``[H, W, 3]`` -> ``[3, dst_h, dst_w]`` with the reference's sampling rule:
    source coordinate ``(d + 0.5) * ratio - 0.5``, lower index ``max(0, trunc)``, upper index
    clamped to the edge, weights taken from the unclamped fraction."""
    H, W, _ = rgb.shape

    def axis(n_src: int, n_dst: int):
        src = (torch.arange(n_dst, dtype=torch.float64) + 0.5) * (n_src / n_dst) - 0.5
        i0 = src.trunc().clamp_min(0).long()
        i1 = (i0 + 1).clamp_max(n_src - 1)
        return i0, i1, (src - i0.double())
    y0, y1, fy = axis(H, dst_h)
    x0, x1, fx = axis(W, dst_w)
    p = rgb.permute(2, 0, 1).double()
    fy, fx = fy.view(1, -1, 1), fx.view(1, 1, -1)
    top = p[:, y0][:, :, x0] * (1 - fx) + p[:, y0][:, :, x1] * fx
    bot = p[:, y1][:, :, x0] * (1 - fx) + p[:, y1][:, :, x1] * fx
    return (top * (1 - fy) + bot * fy).float()


def _normalized_half(path: str, w: int, h: int) -> torch.Tensor:
    """Composite on white, scale to [-1, 1] (mean = std = 0.5), resize, clamp: ``[3, h, w]``."""
    rgb = composite_over_white(decode_image_rgba(path)) / 255.0
    rgb = (rgb - 0.5) / 0.5
    return resize_bilinear_chw(rgb, w, h).clamp_(-1.0, 1.0)


class Gemma3ImageProcessor:
    START_OF_IMAGE, END_OF_IMAGE, NEWLINE_NEWLINE, PAD = 255999, 256000, 108, 0

    def __init__(self, tokens_per_image: int = 256, image_size: int = 896, patch_size: int = 14):
        self.tokens_per_image, self.image_size, self.patch_size = tokens_per_image, image_size, patch_size

    def process(self, path: str) -> torch.Tensor:
        return _normalized_half(path, self.image_size, self.image_size)


class Gemma4ImageProcessor:
    def __init__(self, patch_size: int = 16, n_merge: int = 3, min_tokens: int = 40, max_tokens: int = 280):
        self.patch_size, self.n_merge = patch_size, n_merge
        area = patch_size * patch_size * n_merge * n_merge
        self.min_pixels, self.max_pixels = min_tokens * area, max_tokens * area

    def smart_resize(self, w: int, h: int) -> Tuple[int, int]:
        align = self.patch_size * self.n_merge
        total = w * h
        if self.max_pixels > 0 and total > 0:
            f = math.sqrt(self.max_pixels / total)
            return (max(align, int(math.floor(f * w / align)) * align), max(align, int(math.floor(f * h / align)) * align))
        return max(align, (w // align) * align), max(align, (h // align) * align)

    def output_tokens(self, w: int, h: int) -> int:
        return (w // self.patch_size // self.n_merge) * (h // self.patch_size // self.n_merge)

    def process(self, path: str):
        w0, h0 = read_image_dimensions(path)
        w, h = self.smart_resize(w0, h0)
        return _normalized_half(path, w, h), w, h


def _round_half_even(x: float) -> int:
    return int(round(x))


class Qwen35ImageProcessor:
    def __init__(self, patch_size: int = 14, merge_size: int = 2, shortest_edge: int = 64 * 1024,
                 longest_edge: int = 2 * 1024 * 1024):
        self.patch_size, self.merge_size = patch_size, merge_size
        self.factor = patch_size * merge_size
        self.shortest_edge, self.longest_edge = shortest_edge, longest_edge

    def smart_resize(self, height: int, width: int) -> Tuple[int, int]:
        f = self.factor
        if height < f or width < f:
            raise ValueError(f"Image too small: {height}x{width}, minimum {f}x{f}")
        hb, wb = _round_half_even(height / f) * f, _round_half_even(width / f) * f
        if hb * wb > self.longest_edge:
            beta = math.sqrt(height * width / self.longest_edge)
            hb, wb = int(math.floor(height / beta / f)) * f, int(math.floor(width / beta / f)) * f
        elif hb * wb < self.shortest_edge:
            beta = math.sqrt(self.shortest_edge / (height * width))
            hb, wb = int(math.ceil(height * beta / f)) * f, int(math.ceil(width * beta / f)) * f
        return hb, wb

    def image_token_count(self, height: int, width: int) -> int:
        h, w = self.smart_resize(height, width)
        return (h // self.patch_size // self.merge_size) * (w // self.patch_size // self.merge_size)

    def process(self, path: str):
        w0, h0 = read_image_dimensions(path)
        h, w = self.smart_resize(h0, w0)
        return _normalized_half(path, w, h), h, w


class Mistral3ImageProcessor:
    IMG, IMG_BREAK, IMG_END = 10, 12, 13
    MEAN = (0.48145466, 0.4578275, 0.40821073)
    STD = (0.26862954, 0.26130258, 0.27577711)

    def __init__(self, image_size: int = 1540, patch_size: int = 14, longest_edge: int = 1540):
        self.image_size, self.patch_size, self.longest_edge = image_size, patch_size, longest_edge

    def target_size(self, w: int, h: int) -> Tuple[int, int]:
        ratio = max(h / self.longest_edge, w / self.longest_edge)
        if ratio > 1.0:
            w, h = int(math.floor(w / ratio)), int(math.floor(h / ratio))
        P = self.patch_size
        return ((w - 1) // P + 1) * P, ((h - 1) // P + 1) * P

    def vision_token_count(self, w: int, h: int, merge: int) -> int:
        mw, mh = w // self.patch_size // merge, h // self.patch_size // merge
        return mw * mh + mh

    def process(self, path: str):
        rgba = decode_image_rgba(path)
        h0, w0 = rgba.shape[:2]
        w, h = self.target_size(w0, h0)
        rgb = resize_bilinear_chw(composite_over_white(rgba) / 255.0, w, h)
        mean = torch.tensor(self.MEAN).view(3, 1, 1)
        std = torch.tensor(self.STD).view(3, 1, 1)
        return (rgb - mean) / std, w, h
