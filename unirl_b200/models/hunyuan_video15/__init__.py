"""HunyuanVideo 1.5: 54 joint blocks, 32-channel latents.  Parity: ``unirl/models/hunyuan_video15/``."""
from unirl_b200.models.hunyuan_video15.pipeline import HunyuanVideo15Bundle, HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig

from unirl_b200.models.dit.conditions import DiTConditions as HunyuanVideo15Conditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["HunyuanVideo15Conditions", "HunyuanVideo15Bundle", "HunyuanVideo15Pipeline", "HunyuanVideo15PipelineConfig"]
