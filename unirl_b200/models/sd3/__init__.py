"""Stable Diffusion 3 / 3.5 (MMDiT) on the generic DiT core.  Parity: ``unirl/models/sd3/``."""
from unirl_b200.models.sd3.bundle import SD3Bundle
from unirl_b200.models.sd3.config import SD3PipelineConfig
from unirl_b200.models.sd3.conditions import SD3Conditions
from unirl_b200.models.sd3.diffusion import SD3DiffusionParams, SD3DiffusionStage
from unirl_b200.models.sd3.pipeline import SD3Pipeline

__all__ = ["SD3Bundle", "SD3PipelineConfig", "SD3Conditions", "SD3DiffusionParams", "SD3DiffusionStage", "SD3Pipeline"]
