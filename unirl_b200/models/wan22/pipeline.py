"""WAN 2.2 — a high-noise and a low-noise expert with identical geometry; a step uses the high-noise expert while
``timestep ≥ boundary·1000`` and the low-noise expert afterwards.  Both experts are trainable modules of the bundle
(the sharded trainer builds one group set per expert).  Parity: ``unirl/models/wan22/diffusion.py``, ``wan22/bundle.py``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from unirl_b200.models.dit.modeling import DiTTransformer
from unirl_b200.models.wan21.pipeline import Wan21Bundle, Wan21Pipeline, Wan21PipelineConfig


@dataclass
class Wan22PipelineConfig(Wan21PipelineConfig):
    boundary_ratio: float = 0.875
    clip_vision: bool = False  # the 2.2 image-to-video checkpoints condition on the first frame's latents only
    num_train_timesteps: int = 1000  # the time scale the boundary is expressed on (σ · num_train_timesteps is what the experts see)


class WanDualTransformer(nn.Module):
    block_class_names = DiTTransformer.block_class_names
    _no_split_modules = DiTTransformer._no_split_modules

    def __init__(self, high: DiTTransformer, low: DiTTransformer, boundary_ratio: float):
        super().__init__()
        self.high_noise, self.low_noise, self.boundary = high, low, float(boundary_ratio) * 1000.0
        self.cfg = high.cfg

    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, *a: Any, **k: Any) -> torch.Tensor:
        t = float(timestep.reshape(-1)[0])  # a denoising step uses one noise level for the whole batch
        return (self.high_noise if t >= self.boundary else self.low_noise)(latents, timestep, *a, **k)


class Wan22Bundle(Wan21Bundle):
    @classmethod
    def from_config(cls, config: Wan22PipelineConfig, sp: Optional[Any] = None) -> "Wan22Bundle":
        b = super().from_config(config, sp)
        low = DiTTransformer(b.spec.transformer, dtype=next(b.transformer.parameters()).dtype, device=next(b.transformer.parameters()).device,
                             gradient_checkpointing=config.use_gradient_checkpointing, sp=sp).init_weights(config.init_seed + 13)
        b.transformer = WanDualTransformer(b.transformer, low, config.boundary_ratio)
        return b

    def trainable_modules(self) -> Dict[str, nn.Module]:
        return {"transformer": self.transformer}


class Wan22Pipeline(Wan21Pipeline):
    @classmethod
    def from_config(cls, config: Wan22PipelineConfig) -> "Wan22Pipeline":
        return cls(Wan22Bundle.from_config(config))


__all__ = ["Wan22PipelineConfig", "WanDualTransformer", "Wan22Bundle", "Wan22Pipeline"]
