"""Image → flattened patch tensor in the layout the vision tower consumes (the job of the HF image processor).

An image ``[3, H, W]`` in ``[0, 1]`` is resized so both sides are multiples of ``patch·merge`` within the pixel budget,
normalised, repeated ``temporal_patch`` times along time, cut into ``patch x patch`` patches and ordered so that every
``merge x merge`` group of neighbouring patches is contiguous.  Returns ``(pixel_values [t·h·w, C·tp·p·p], grid (t, h, w))``.
"""

from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn.functional as F

from unirl_b200.models.qwen_vl.modeling import VisionConfig

_MEAN = torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(3, 1, 1)
_STD = torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(3, 1, 1)


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    hb, wb = max(factor, round(h / factor) * factor), max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb, wb = max(factor, math.floor(h / beta / factor) * factor), max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


def preprocess_image(img: torch.Tensor, c: VisionConfig, min_pixels: int, max_pixels: int) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    p, ms, tp = c.patch_size, c.spatial_merge_size, c.temporal_patch_size
    hb, wb = smart_resize(img.shape[-2], img.shape[-1], p * ms, min_pixels, max_pixels)
    x = F.interpolate(img.float().unsqueeze(0), size=(hb, wb), mode="bicubic", align_corners=False).squeeze(0).clamp(0, 1)
    x = (x - _MEAN) / _STD
    gh, gw = hb // p, wb // p
    x = x.unsqueeze(0).expand(tp, -1, -1, -1)  # a still image fills one temporal patch
    x = x.reshape(1, tp, 3, gh // ms, ms, p, gw // ms, ms, p).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(gh * gw, 3 * tp * p * p), (1, gh, gw)


__all__ = ["smart_resize", "preprocess_image"]
