"""HunyuanVideo: 20 double + 40 single blocks, guidance embedding, LLM + CLIP text.  Parity: ``unirl/models/hunyuan_video/``."""
from unirl_b200.models.hunyuan_video.pipeline import HunyuanVideoBundle, HunyuanVideoPipeline, HunyuanVideoPipelineConfig

__all__ = ["HunyuanVideoBundle", "HunyuanVideoPipeline", "HunyuanVideoPipelineConfig"]
