"""HunyuanVideo 1.5: 54 joint blocks, 32-channel latents — config, bundle and pipeline on the generic DiT core.  Parity: ``unirl/models/hunyuan_video15/``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class HunyuanVideo15PipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-video15"


class HunyuanVideo15Bundle(DiTBundle):
    pass


class HunyuanVideo15Pipeline(DiTPipeline):
    def __init__(self, bundle):
        super().__init__(bundle)
        pass

    @classmethod
    def from_config(cls, config: HunyuanVideo15PipelineConfig) -> "HunyuanVideo15Pipeline":
        return cls(HunyuanVideo15Bundle.from_config(config))


__all__ = ["HunyuanVideo15PipelineConfig", "HunyuanVideo15Bundle", "HunyuanVideo15Pipeline"]
