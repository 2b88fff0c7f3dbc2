"""Unified text + image transformer (shared by the HunyuanImage-3 and Bagel packages)."""
from unirl_b200.models.unified.modeling import MoEFFN, UnifiedConfig, UnifiedTransformer
from unirl_b200.models.unified.pipeline import UnifiedBundle, UnifiedPipeline, UnifiedPipelineConfig
from unirl_b200.models.unified.stages import UnifiedARStage, UnifiedConditions, UnifiedDiffusionStage

__all__ = ["MoEFFN", "UnifiedConfig", "UnifiedTransformer", "UnifiedBundle", "UnifiedPipeline", "UnifiedPipelineConfig", "UnifiedARStage", "UnifiedConditions",
           "UnifiedDiffusionStage"]
