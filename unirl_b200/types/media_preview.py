"""``MediaPreview`` — a few down-scaled decoded samples kept for logging after the heavy decoded
media is dropped from the training payload.  Parity: ``unirl/types/media_preview.py`` (``MediaPreview``
``:25``, ``build_media_preview_for_track`` ``:130``)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, shared_field


@dataclass
class MediaPreview(Batch):
    kind: str = shared_field(default="image")
    thumbs: Optional[torch.Tensor] = concat_field(default=None)  # uint8 [n, C, h, w] (image) / [n, F, C, h, w] (video)
    captions: List[str] = concat_field(default_factory=list)
    sample_ids: List[str] = concat_field(default_factory=list)


def _thumb(x: torch.Tensor, side: int) -> torch.Tensor:
    x = x.detach().float().clamp(0, 1)
    flat = x.reshape(-1, *x.shape[-3:])
    flat = torch.nn.functional.interpolate(flat, size=(side, side), mode="bilinear", align_corners=False)
    return (flat * 255).round().to(torch.uint8).reshape(*x.shape[:-2], side, side).cpu()


def build_media_preview_for_track(track: Any, max_items: int = 8, side: int = 128, captions: Optional[List[str]] = None) -> Optional[MediaPreview]:
    """Thumbnail the first ``max_items`` decoded samples of ``track`` (``None`` if nothing decodable)."""
    dec = getattr(track, "decoded", None)
    if dec is None:
        return None
    n = min(max_items, len(dec))
    if n == 0:
        return None
    ids = list(track.sample_ids[:n])
    caps = list((captions or [""] * n)[:n])
    if hasattr(dec, "pixels") and isinstance(dec.pixels, torch.Tensor):
        return MediaPreview(kind="image", thumbs=_thumb(dec.pixels[:n], side), captions=caps, sample_ids=ids)
    if hasattr(dec, "frames") and isinstance(dec.frames, torch.Tensor) and dec.cu_seqlens is not None:
        cu = dec.cu_seqlens.tolist()
        f = min(cu[i + 1] - cu[i] for i in range(n))
        vids = torch.stack([dec.frames[cu[i] : cu[i] + f] for i in range(n)])
        return MediaPreview(kind="video", thumbs=_thumb(vids, side), captions=caps, sample_ids=ids)
    if hasattr(dec, "texts"):
        return MediaPreview(kind="text", thumbs=None, captions=list(dec.texts[:n]), sample_ids=ids)
    return None


__all__ = ["MediaPreview", "build_media_preview_for_track"]
