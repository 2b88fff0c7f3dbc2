"""``SD3Pipeline`` — prompts → images; ``latent_shape = (16, H/8, W/8)`` (``unirl/models/sd3/pipeline.py:97-203``)."""
from __future__ import annotations

from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.sd3.bundle import SD3Bundle
from unirl_b200.models.sd3.config import SD3PipelineConfig


class SD3Pipeline(DiTPipeline):
    @classmethod
    def from_config(cls, config: SD3PipelineConfig) -> "SD3Pipeline":
        return cls(SD3Bundle.from_config(config))


__all__ = ["SD3Pipeline"]
