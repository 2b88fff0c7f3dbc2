"""``LatentSegment`` — denoising trajectories ``[N, K, …]`` plus dense per-SDE-step log-probs.

``sde_logp[:, s]`` is the element-mean Gaussian log-prob of the transition at step
``sde_indices[s]``; ``sde_means`` the matching transition means (Flow-DPPO's anchor).  Either the
rollout engine fills them (the native sampler's fused SDE kernel emits both for free) or the
algorithm's ``prepare_segment`` recomputes them.  Parity: ``unirl/types/segments/latent.py:40-135``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from unirl_b200.distributed.tensor.batch import concat_field, shared_field
from unirl_b200.types.conditions.base import Condition, Modality
from unirl_b200.types.conditions.image import ImageLatentCondition
from unirl_b200.types.segments.base import Segment


@dataclass
class LatentSegment(Segment):
    modality: Modality = shared_field(default=Modality.IMAGE)  # instance field: survives select/slice/concat

    latents: Optional[torch.Tensor] = concat_field(default=None)
    sigmas: Optional[torch.Tensor] = shared_field(default=None)
    indices: Optional[torch.Tensor] = shared_field(default=None)
    sde_logp: Optional[torch.Tensor] = concat_field(default=None)
    sde_means: Optional[torch.Tensor] = concat_field(default=None)
    sde_indices: Optional[torch.Tensor] = shared_field(default=None)
    log_probs: Optional[torch.Tensor] = concat_field(default=None)
    loss_mask: Optional[torch.Tensor] = concat_field(default=None)

    def as_condition(self) -> Optional[Condition]:
        if self.modality is not Modality.IMAGE or self.latents is None:
            return None
        return ImageLatentCondition(latents=self.latents[:, -1])

    def slot_of(self, step_idx: int) -> int:
        if self.indices is None:
            raise RuntimeError("LatentSegment has no stored-position index")
        hit = (self.indices == int(step_idx)).nonzero().flatten()
        if not hit.numel():
            raise KeyError(f"step {step_idx} is not stored (stored: {self.indices.tolist()})")
        return int(hit[0])

    def latents_at(self, step_idx: int) -> torch.Tensor:
        if self.latents is None:
            raise RuntimeError("LatentSegment has no latents")
        return self.latents[:, self.slot_of(step_idx)]


def make_image_segment(**kw) -> LatentSegment:
    return LatentSegment(modality=Modality.IMAGE, **kw)


def make_video_segment(**kw) -> LatentSegment:
    return LatentSegment(modality=Modality.VIDEO, **kw)


def make_audio_segment(**kw) -> LatentSegment:
    return LatentSegment(modality=Modality.AUDIO, **kw)


__all__ = ["LatentSegment", "make_image_segment", "make_video_segment", "make_audio_segment"]
