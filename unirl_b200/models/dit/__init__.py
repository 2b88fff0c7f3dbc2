"""Generic DiT core shared by every diffusion model family (see ``modeling.py`` for the block zoo)."""
from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import PRESETS, DiTPipelineConfig, FamilySpec, resolve_family
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage
from unirl_b200.models.dit.modeling import DiTConfig, DiTTransformer
from unirl_b200.models.dit.pipeline import DiTPipeline

__all__ = ["DiTBundle", "DiTConditions", "DiTPipelineConfig", "FamilySpec", "PRESETS", "resolve_family", "DiTDiffusionParams", "DiTDiffusionStage",
           "DiTConfig", "DiTTransformer", "DiTPipeline"]
