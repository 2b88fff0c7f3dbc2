"""Z-Image: single-stream DiT over the concatenated text + latent sequence — config, bundle and pipeline on the generic DiT core.  Parity: ``unirl/models/z_image/``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class ZImagePipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:z-image"


class ZImageBundle(DiTBundle):
    pass


class ZImagePipeline(DiTPipeline):
    def __init__(self, bundle):
        super().__init__(bundle)
        pass

    @classmethod
    def from_config(cls, config: ZImagePipelineConfig) -> "ZImagePipeline":
        return cls(ZImageBundle.from_config(config))


__all__ = ["ZImagePipelineConfig", "ZImageBundle", "ZImagePipeline"]
