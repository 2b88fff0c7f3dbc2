"""Qwen-Image: 60 joint blocks, packed 2x2 latents, LLM text tower, dynamic shift, CFG norm correction.  Parity: ``unirl/models/qwen_image/``."""
from unirl_b200.models.qwen_image.pipeline import QwenImageBundle, QwenImagePipeline, QwenImagePipelineConfig

__all__ = ["QwenImageBundle", "QwenImagePipeline", "QwenImagePipelineConfig"]
