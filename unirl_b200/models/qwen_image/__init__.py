"""Qwen-Image: 60 joint blocks, packed 2x2 latents, LLM text tower, dynamic shift, CFG norm correction.  Parity: ``unirl/models/qwen_image/``."""
from unirl_b200.models.qwen_image.pipeline import QwenImageBundle, QwenImagePipeline, QwenImagePipelineConfig

from unirl_b200.models.dit.conditions import DiTConditions as QwenImageConditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["QwenImageConditions", "QwenImageBundle", "QwenImagePipeline", "QwenImagePipelineConfig"]
