"""Construction config of the Qwen2.5-VL pipeline (``unirl/models/qwen_vl/config.py`` field names)."""

from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.qwen3.config import Qwen3PipelineConfig


@dataclass
class QwenVLPipelineConfig(Qwen3PipelineConfig):
    pretrained_model_ckpt_path: str = "random:tiny-vl"
    min_pixels: int = 4 * 28 * 28
    max_pixels: int = 1280 * 28 * 28
    freeze_vision_tower: bool = False  # True: the vision tower takes no gradient (the reference's default); only the decoder is trained


__all__ = ["QwenVLPipelineConfig"]
