"""Qwen2.5-VL (vision-language AR policy).  Parity: ``unirl/models/qwen_vl/``."""
from unirl_b200.models.qwen_vl.ar import QwenVLARStage
from unirl_b200.models.qwen_vl.bundle import QwenVLBundle
from unirl_b200.models.qwen_vl.conditions import QwenVLARConditions
from unirl_b200.models.qwen_vl.config import QwenVLPipelineConfig
from unirl_b200.models.qwen_vl.modeling import QwenVLConfig, QwenVLTransformer
from unirl_b200.models.qwen_vl.pipeline import QwenVLPipeline

__all__ = ["QwenVLARStage", "QwenVLBundle", "QwenVLARConditions", "QwenVLPipelineConfig", "QwenVLConfig", "QwenVLTransformer", "QwenVLPipeline"]
