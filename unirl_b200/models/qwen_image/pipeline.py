"""Qwen-Image: 60 joint blocks, packed 2x2 latents, LLM text tower, dynamic shift, CFG norm correction — config, bundle and pipeline on the generic DiT core.  Parity: ``unirl/models/qwen_image/``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class QwenImagePipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:qwen-image"


class QwenImageBundle(DiTBundle):
    pass


class QwenImageDiffusionStage(DiTDiffusionStage):
    """CFG with norm correction: the guided prediction is rescaled to the norm of the conditional one (per token)."""

    def _guided(self, v_uncond, v_cond, p):
        vg = v_uncond + p.guidance_scale * (v_cond - v_uncond)
        nc, ng = v_cond.norm(dim=1, keepdim=True), vg.norm(dim=1, keepdim=True).clamp_min(1e-12)
        return vg * (nc / ng)


class QwenImagePipeline(DiTPipeline):
    def __init__(self, bundle):
        super().__init__(bundle)
        self.diffusion = QwenImageDiffusionStage(bundle, bundle.spec.default_strategy, bundle.config.autocast_precision)

    @classmethod
    def from_config(cls, config: QwenImagePipelineConfig) -> "QwenImagePipeline":
        return cls(QwenImageBundle.from_config(config))


__all__ = ["QwenImagePipelineConfig", "QwenImageBundle", "QwenImagePipeline"]
