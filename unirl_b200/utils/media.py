"""Tensors → PIL previews, free of any logging dependency (the loggers build their own media objects from these).

``[C, H, W]`` frames in ``[0, 1]``; a batch of videos ``[B, C, F, H, W]`` is previewed by its middle frame.
Parity: ``unirl/utils/media.py`` (``tensor_frame_to_pil``, ``tensor_to_pil``).
"""

from __future__ import annotations

from typing import Any, List

import torch


def tensor_frame_to_pil(frame: torch.Tensor) -> Any:
    from PIL import Image

    if frame.dim() != 3:
        raise ValueError(f"a [C, H, W] frame is expected, got {tuple(frame.shape)}")
    x = frame.detach().to(torch.float32).cpu().clamp_(0.0, 1.0)
    if x.shape[0] == 1:
        x = x.expand(3, -1, -1)
    return Image.fromarray((x.permute(1, 2, 0) * 255.0).round().to(torch.uint8).numpy())


def tensor_to_pil(images: torch.Tensor) -> List[Any]:
    """``[B, C, H, W]`` images or ``[B, C, F, H, W]`` videos → one preview per sample."""
    x = images.detach().cpu()
    if x.dim() == 5:
        x = x[:, :, x.shape[2] // 2]
    if x.dim() != 4:
        raise ValueError(f"[B, C, H, W] or [B, C, F, H, W] expected, got {tuple(images.shape)}")
    return [tensor_frame_to_pil(f) for f in x]


__all__ = ["tensor_frame_to_pil", "tensor_to_pil"]
