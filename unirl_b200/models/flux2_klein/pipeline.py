"""FLUX.2 klein — config, bundle (empirical-μ schedule policy) and pipeline.  Parity: ``unirl/models/flux2_klein/``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.flux2_klein.schedule import KleinSchedulePolicy


@dataclass
class Flux2KleinPipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:flux2-klein"


class Flux2KleinBundle(DiTBundle):
    def schedule_policy(self) -> KleinSchedulePolicy:
        t = self.spec.transformer
        return KleinSchedulePolicy(shift=float(self.config.shift if self.config.shift is not None else self.spec.shift),
                                   vae_scale_factor=t.vae_scale_factor, patch_size=2 * t.patch_size[-1])


class Flux2KleinPipeline(DiTPipeline):
    @classmethod
    def from_config(cls, config: Flux2KleinPipelineConfig) -> "Flux2KleinPipeline":
        return cls(Flux2KleinBundle.from_config(config))


__all__ = ["Flux2KleinPipelineConfig", "Flux2KleinBundle", "Flux2KleinPipeline"]
