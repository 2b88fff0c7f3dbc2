"""Z-Image: single-stream DiT over the concatenated text + latent sequence, on the generic DiT core.

What the family changes against the core conventions (``unirl/models/z_image/diffusion.py:84-141``):

* the transformer is conditioned on ``1 − σ`` (time runs the other way), and its output is the NEGATED flow velocity;
* classifier-free guidance is on whenever ``guidance_scale > 0`` and a negative prompt exists, and combines as
  ``cond + g·(cond − uncond)`` (a scale of ``g`` there is ``1 + g`` in the usual ``uncond + s·(cond − uncond)`` form);
* captions have their own lengths: padding is masked out of the joint sequence (``text.attn_mask``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline


@dataclass
class ZImagePipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:z-image"


class ZImageBundle(DiTBundle):
    pass


class ZImageDiffusionStage(DiTDiffusionStage):
    def _branches(self, x: torch.Tensor, sigma: torch.Tensor, cond: DiTConditions, p: DiTDiffusionParams) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        model = self.bundle.transformer
        t = (1.0 - sigma.to(x.device).float().reshape(-1)).expand(x.shape[0]) * 1000.0
        txt, neg = cond.text, cond.negative_text
        if not (p.guidance_scale > 0.0 and neg is not None):
            return -model(x, t, txt.embeds, txt.pooled, txt.attn_mask).float(), None
        width = max(txt.embeds.shape[1], neg.embeds.shape[1])
        pad = lambda e: torch.nn.functional.pad(e, (0, 0, 0, width - e.shape[1]))  # noqa: E731
        ones = lambda c: torch.ones(c.embeds.shape[:2], dtype=torch.long, device=c.embeds.device) if c.attn_mask is None else c.attn_mask  # noqa: E731
        padm = lambda c: torch.nn.functional.pad(ones(c), (0, width - c.embeds.shape[1]))  # noqa: E731
        v = -model(torch.cat([x, x]), torch.cat([t, t]), torch.cat([pad(neg.embeds), pad(txt.embeds)]), None, torch.cat([padm(neg), padm(txt)])).float()
        vu, vc = v.chunk(2)
        return vc, vu

    def _guided(self, v_uncond: torch.Tensor, v_cond: torch.Tensor, p: DiTDiffusionParams) -> torch.Tensor:
        return v_cond + p.guidance_scale * (v_cond - v_uncond)


class ZImagePipeline(DiTPipeline):
    def __init__(self, bundle, **options):
        super().__init__(bundle, **options)
        self.diffusion = ZImageDiffusionStage(bundle, bundle.spec.default_strategy, bundle.config.autocast_precision)

    @classmethod
    def from_config(cls, config: ZImagePipelineConfig) -> "ZImagePipeline":
        return cls(ZImageBundle.from_config(config))


__all__ = ["ZImagePipelineConfig", "ZImageBundle", "ZImageDiffusionStage", "ZImagePipeline"]
