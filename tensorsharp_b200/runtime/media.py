"""Media helpers: video frame sampling policy, frame extraction, image loading.

Parity: TensorSharp.Models/MediaHelper.cs:19-35 (VIDEO_MAX_FRAMES, default 4), :37-80
(ExtractVideoFrames: candidates at ``fps`` frames per second, then evenly spaced), :82-117
(SelectEvenlySpacedIndices).  Decoding uses OpenCV / Pillow when importable; without them the
functions raise a clear error rather than guessing.
"""
from __future__ import annotations

import os
import tempfile
import uuid
from typing import List

DEFAULT_VIDEO_MAX_FRAMES = 4


def get_configured_max_video_frames(fallback: int = DEFAULT_VIDEO_MAX_FRAMES) -> int:
    raw = os.environ.get("VIDEO_MAX_FRAMES")
    if raw and raw.strip():
        try:
            v = int(raw)
            if v > 0:
                return v
        except ValueError:
            pass
    return fallback if fallback > 0 else DEFAULT_VIDEO_MAX_FRAMES


def _round_half_even(x: float) -> int:
    return int(round(x))            # Python rounds half to even, as .NET's Math.Round does


def select_evenly_spaced_indices(count: int, max_count: int) -> List[int]:
    if count <= 0 or max_count <= 0:
        return []
    if count <= max_count:
        return list(range(count))
    if max_count == 1:
        return [count // 2]
    step = (count - 1) / (max_count - 1)
    out: List[int] = []
    prev = -1
    for i in range(max_count):
        idx = _round_half_even(i * step)
        if idx <= prev:
            idx = prev + 1
        if idx >= count:
            idx = count - 1
        out.append(idx)
        prev = idx
    return out


def extract_video_frames(video_path: str, max_frames: int = 0, fps: float = 1.0) -> List[str]:
    """Write up to ``max_frames`` PNG frames of the video into a fresh temp directory."""
    try:
        import cv2
    except ImportError as e:                                       # pragma: no cover
        raise RuntimeError("video upload needs OpenCV (cv2), which is not importable here") from e
    if max_frames <= 0:
        max_frames = get_configured_max_video_frames()
    out_dir = os.path.join(tempfile.gettempdir(), f"frames_{uuid.uuid4().hex}")
    os.makedirs(out_dir, exist_ok=True)
    cap = cv2.VideoCapture(video_path)
    try:
        if not cap.isOpened():
            raise RuntimeError(f"Failed to open video file: {video_path}")
        vfps = cap.get(cv2.CAP_PROP_FPS)
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        if vfps <= 0 or total <= 0:
            raise RuntimeError(f"Invalid video: fps={vfps}, frames={total}")
        interval = max(1, _round_half_even(vfps / fps))
        cand = list(range(0, total, interval))
        frames: List[str] = []
        for pos in select_evenly_spaced_indices(len(cand), max_frames):
            cap.set(cv2.CAP_PROP_POS_FRAMES, cand[pos])
            ok, mat = cap.read()
            if not ok or mat is None or mat.size == 0:
                break
            path = os.path.join(out_dir, f"frame_{len(frames) + 1:04d}.png")
            cv2.imwrite(path, mat)
            frames.append(path)
        return frames
    finally:
        cap.release()


def load_image_rgb(path: str):
    """Decode an image file to a uint8 ``[H, W, 3]`` torch tensor (alpha composited on white:
    Gemma3ImageProcessor.cs / Qwen35ImageProcessor.cs do the same before resizing)."""
    import numpy as np
    import torch
    from PIL import Image
    with Image.open(path) as im:
        if im.mode in ("RGBA", "LA", "P"):
            im = im.convert("RGBA")
            bg = Image.new("RGBA", im.size, (255, 255, 255, 255))
            im = Image.alpha_composite(bg, im).convert("RGB")
        else:
            im = im.convert("RGB")
        return torch.from_numpy(np.array(im, dtype=np.uint8))
