"""HunyuanVideo: 20 double + 40 single blocks, guidance embedding, LLM + CLIP text — config, bundle and pipeline on the generic DiT core.  Parity: ``unirl/models/hunyuan_video/``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class HunyuanVideoPipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-video"


class HunyuanVideoBundle(DiTBundle):
    pass


class HunyuanVideoPipeline(DiTPipeline):
    def __init__(self, bundle):
        super().__init__(bundle)
        pass

    @classmethod
    def from_config(cls, config: HunyuanVideoPipelineConfig) -> "HunyuanVideoPipeline":
        return cls(HunyuanVideoBundle.from_config(config))


__all__ = ["HunyuanVideoPipelineConfig", "HunyuanVideoBundle", "HunyuanVideoPipeline"]
