"""SD3 diffusion stage: CFG as one ``[uncond, cond]`` batch, CPS transition by default (``unirl/models/sd3/diffusion.py:41-133``)."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage


@dataclass
class SD3DiffusionParams(DiTDiffusionParams):
    guidance_scale: float = 4.5


class SD3DiffusionStage(DiTDiffusionStage):
    def __init__(self, bundle, autocast_precision: str = "bf16"):
        super().__init__(bundle, "cps", autocast_precision)


__all__ = ["SD3DiffusionParams", "SD3DiffusionStage"]
