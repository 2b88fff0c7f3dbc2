"""HunyuanVideo 1.5: 54 joint blocks, 32-channel latents.  Parity: ``unirl/models/hunyuan_video15/``."""
from unirl_b200.models.hunyuan_video15.pipeline import HunyuanVideo15Bundle, HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig

__all__ = ["HunyuanVideo15Bundle", "HunyuanVideo15Pipeline", "HunyuanVideo15PipelineConfig"]
