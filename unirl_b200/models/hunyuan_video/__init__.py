"""HunyuanVideo: 20 double + 40 single blocks, guidance embedding, LLM + CLIP text.  Parity: ``unirl/models/hunyuan_video/``."""
from unirl_b200.models.hunyuan_video.pipeline import HunyuanVideoBundle, HunyuanVideoPipeline, HunyuanVideoPipelineConfig

from unirl_b200.models.dit.conditions import DiTConditions as HunyuanVideoConditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["HunyuanVideoConditions", "HunyuanVideoBundle", "HunyuanVideoPipeline", "HunyuanVideoPipelineConfig"]
