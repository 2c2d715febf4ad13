"""Decoded images and video frames -> the pixel rows a vision tower reads.

``smart_resize`` picks the size closest to the original whose sides are whole numbers of merge blocks
(``patch * merge`` pixels) and whose area lies inside the model's pixel limits.  ``patchify`` rescales to [0, 1],
normalises per channel and cuts the frames into ``[t * h * w, C * Tp * p * p]`` rows in merge-block order: the
``m x m`` patches that the tower's merger folds into one decoder row are consecutive.  A still image is repeated over
the temporal patch; a video's frame count is padded to a whole number of temporal patches with its last frame.

Decoding (``decode_image``) uses Pillow on bytes that the media resolver has already sniffed and bounded.

Reference counterpart: ``models/qwen3_5/multimodal.py:1093-1120`` (``_smart_resize``), ``:1278-1358`` (``_patchify``).
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass

import numpy as np


class VisionInputError(ValueError):
    pass


@dataclass(frozen=True)
class PatchGeometry:
    patch_size: int = 16
    merge_size: int = 2
    temporal_patch_size: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 28 * 28 * 1280
    mean: tuple[float, ...] = (0.5, 0.5, 0.5)
    std: tuple[float, ...] = (0.5, 0.5, 0.5)

    @property
    def factor(self) -> int:
        return self.patch_size * self.merge_size


@dataclass
class MediaPatches:
    pixels: np.ndarray                  # float32 [t * h * w, C * Tp * p * p]
    grid: tuple[int, int, int]          # (t, h, w) in patches

    def rows(self, merge: int) -> int:
        t, h, w = self.grid
        return t * h * w // (merge * merge)


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    if height <= 0 or width <= 0:
        raise VisionInputError("image sides are positive")
    if max(height, width) / min(height, width) > 200:
        raise VisionInputError("aspect ratio above 200")
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


def decode_image(data: bytes, max_side: int = 16384):
    """Bytes -> RGB ``PIL.Image`` (alpha is composited on white)."""
    from PIL import Image
    try:
        img = Image.open(io.BytesIO(data))
        img.load()
    except Exception as e:                                              # Pillow raises many types on corrupt input
        raise VisionInputError(f"the image cannot be decoded: {type(e).__name__}") from None
    if max(img.size) > max_side:
        raise VisionInputError(f"image side above {max_side} pixels")
    if img.mode in ("RGBA", "LA") or (img.mode == "P" and "transparency" in img.info):
        rgba = img.convert("RGBA")
        bg = Image.new("RGBA", rgba.size, (255, 255, 255, 255))
        img = Image.alpha_composite(bg, rgba)
    return img.convert("RGB")


def _resized_array(img, geo: PatchGeometry, limits: tuple[int, int] | None = None) -> np.ndarray:
    import torch
    lo, hi = limits or (geo.min_pixels, geo.max_pixels)
    h, w = smart_resize(img.height, img.width, geo.factor, lo, hi)
    arr = np.array(img, dtype=np.uint8)
    if (img.height, img.width) != (h, w):
        # antialiased bicubic on the uint8 image (the result is rounded back to 8 bits, as the image processors the
        # checkpoints were trained with do)
        t = torch.from_numpy(arr).permute(2, 0, 1)[None]
        t = torch.nn.functional.interpolate(t, size=(h, w), mode="bicubic", antialias=True, align_corners=False)
        arr = t[0].permute(1, 2, 0).contiguous().numpy()
    return arr


def patchify_frames(frames: np.ndarray, geo: PatchGeometry) -> MediaPatches:
    """``frames``: uint8 ``[T, H, W, C]`` with H and W whole numbers of merge blocks."""
    if frames.ndim != 4 or frames.dtype != np.uint8 or frames.shape[0] == 0:
        raise VisionInputError("frames are uint8 [T, H, W, C]")
    T, H, W, C = frames.shape
    p, m, tp = geo.patch_size, geo.merge_size, geo.temporal_patch_size
    if H % (p * m) or W % (p * m) or C != len(geo.mean):
        raise VisionInputError("frame sides are whole merge blocks and channels match the normalisation")
    x = frames.astype(np.float32) * np.float32(1 / 255)
    x = (x - np.asarray(geo.mean, np.float32)) / np.asarray(geo.std, np.float32)
    if T % tp:
        x = np.concatenate([x, np.repeat(x[-1:], tp - T % tp, 0)], 0)
    gt, gh, gw = x.shape[0] // tp, H // p, W // p
    x = x.transpose(0, 3, 1, 2)                                        # [T, C, H, W]
    x = x.reshape(gt, tp, C, gh // m, m, p, gw // m, m, p)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                          # gt, gh/m, gw/m, m, m, C, tp, p, p
    return MediaPatches(np.ascontiguousarray(x.reshape(gt * gh * gw, C * tp * p * p)), (gt, gh, gw))


def patchify_image(img, geo: PatchGeometry) -> MediaPatches:
    """One still image (``PIL.Image`` or uint8 ``[H, W, C]``)."""
    if isinstance(img, np.ndarray):
        from PIL import Image
        img = Image.fromarray(img)
    arr = _resized_array(img, geo)
    return patchify_frames(np.repeat(arr[None], geo.temporal_patch_size, 0), geo)


def patchify_video(frames: list, geo: PatchGeometry, max_frames: int = 768, total_pixels: int | None = None) -> MediaPatches:
    """Frames of one clip (``PIL.Image`` each, same size).  Every frame gets the same target size; the pixel budget of
    the whole clip (``total_pixels``) bounds the per-frame area."""
    if not frames or len(frames) > max_frames:
        raise VisionInputError(f"a clip has between 1 and {max_frames} frames")
    size = frames[0].size
    if any(f.size != size for f in frames):
        raise VisionInputError("frames of a clip share one size")
    hi = geo.max_pixels
    if total_pixels is not None:
        steps = -(-len(frames) // geo.temporal_patch_size)
        hi = max(geo.min_pixels, min(hi, total_pixels // steps))
    arrs = [_resized_array(f, geo, (geo.min_pixels, hi)) for f in frames]
    return patchify_frames(np.stack(arrs), geo)
