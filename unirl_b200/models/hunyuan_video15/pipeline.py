"""HunyuanVideo 1.5: 54 joint blocks, 32-channel latents, on the generic DiT core.

What the family changes (``unirl/models/hunyuan_video15/diffusion.py:37,137-164,46``):

* **channel packing of the transformer input**: ``cat([latents, cond_latents, cond_mask], dim=1)`` -- the conditioning frame latents and a
  one-channel mask ride along with the noisy latents (32 + 32 + 1 = 65 input channels, 32 output channels).  Text-to-video has no
  conditioning frame: both extras are zeros; image-to-video puts the encoded first frame and a mask of ones at frame 0;
* true classifier-free guidance (two branches, ``uncond + g·(cond − uncond)``, no norm correction) whenever ``guidance_scale > 1``;
* two text streams in the reference (a multimodal LLM and a glyph encoder); here the glyph sequence, when a second tower is
  configured, is zero-padded to the LLM width and appended along the token axis.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class HunyuanVideo15PipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-video15"


class HunyuanVideo15Bundle(DiTBundle):
    pass


class HunyuanVideo15DiffusionStage(DiTDiffusionStage):
    def _model_input(self, x: torch.Tensor, cond: DiTConditions) -> torch.Tensor:
        b, _, f, h, w = x.shape
        cond_latents = torch.zeros_like(x)
        cond_mask = torch.zeros(b, 1, f, h, w, dtype=x.dtype, device=x.device)
        img = None if cond.image is None else cond.image.latents
        if img is not None:  # image-to-video: the clean first frame and a mask that marks it
            img = img.to(x)
            img = img if img.dim() == 5 else img.unsqueeze(2)
            cond_latents[:, :, :1] = img[:, :, :1]
            cond_mask[:, :, :1] = 1
        return torch.cat([x, cond_latents, cond_mask], 1)


class HunyuanVideo15Pipeline(DiTPipeline):
    def __init__(self, bundle, **options):
        super().__init__(bundle, **options)
        self.diffusion = HunyuanVideo15DiffusionStage(bundle, bundle.spec.default_strategy, bundle.config.autocast_precision)

    @classmethod
    def from_config(cls, config: HunyuanVideo15PipelineConfig) -> "HunyuanVideo15Pipeline":
        return cls(HunyuanVideo15Bundle.from_config(config))


__all__ = ["HunyuanVideo15PipelineConfig", "HunyuanVideo15Bundle", "HunyuanVideo15DiffusionStage", "HunyuanVideo15Pipeline"]
