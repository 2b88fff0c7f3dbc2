"""SD3 pipeline config: the generic DiT config with SD3.5-Medium defaults (``unirl/models/sd3/config.py``)."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.config import DiTPipelineConfig


@dataclass
class SD3PipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:sd35-medium"
    max_sequence_length: int = 256
    shift: float = 3.0


__all__ = ["SD3PipelineConfig"]
