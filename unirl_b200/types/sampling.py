"""Sampling parameter dataclasses shared by recipes, engines and pipelines.

Parity: ``unirl/types/sampling.py:16-183`` (field names and ``resolve_sde_indices`` precedence:
explicit list > scheduler keyed by rollout id > every step).
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

from unirl_b200.config.require import require


@dataclass
class BaseSamplingParams:
    samples_per_prompt: int = 1


@dataclass
class DiffusionSamplingParams(BaseSamplingParams):
    num_inference_steps: int = 50
    guidance_scale: float = 7.5
    height: int = 256
    width: int = 256
    num_frames: int = 16
    seed: Optional[int] = 42
    init_same_noise: bool = False
    noise_group_ids: Optional[List[str]] = None
    eta: float = 1.0
    sde_strategy: Any = None
    scheduler: Any = None
    sde_indices: Optional[List[int]] = None
    sampler_kwargs: Dict[str, Any] = field(default_factory=dict)
    autocast_precision: str = "bf16"
    trajectory_precision: str = "fp16"
    logprob_precision: str = "fp32"
    max_sequence_length: Optional[int] = None
    taylor_cache_interval: Optional[int] = None
    taylor_cache_order: Optional[int] = None
    distilled_guidance_scale: Optional[float] = None
    guidance_scale_2: Optional[float] = None
    num_samples_per_prompt: int = 1

    def __post_init__(self) -> None:
        if self.num_samples_per_prompt != 1 and self.samples_per_prompt == 1:
            self.samples_per_prompt = self.num_samples_per_prompt
        elif self.samples_per_prompt != 1 and self.num_samples_per_prompt == 1:
            self.num_samples_per_prompt = self.samples_per_prompt
        clash = {f.name for f in fields(self)} - {"sampler_kwargs"}
        clash &= set(self.sampler_kwargs)
        require(not clash, f"sampler_kwargs shadows declared fields {sorted(clash)}")

    def resolve_sde_indices(self, rollout_id: int) -> List[int]:
        if self.sde_indices is not None:
            return [int(i) for i in self.sde_indices]
        if self.scheduler is not None:
            return sorted(self.scheduler.get_sde_indices(int(rollout_id)))
        return list(range(int(self.num_inference_steps)))


@dataclass
class ARSamplingParams(BaseSamplingParams):
    temperature: float = 0.7
    max_new_tokens: int = 512
    top_p: float = 0.9
    top_k: int = 1024
    stop_token_id: Optional[int] = None


@dataclass(kw_only=True)
class ComposedSamplingParams(BaseSamplingParams):
    diffusion: Any
    ar: Any

    def __post_init__(self) -> None:
        self.samples_per_prompt = int(self.diffusion.samples_per_prompt) * int(self.ar.samples_per_prompt)


def get_diffusion_params(sampling: Any) -> Optional[DiffusionSamplingParams]:
    return sampling.diffusion if hasattr(sampling, "diffusion") else sampling


def get_ar_params(sampling: Any) -> Optional[ARSamplingParams]:
    if hasattr(sampling, "ar"):
        return sampling.ar
    return sampling if isinstance(sampling, ARSamplingParams) else None


@dataclass(frozen=True)
class SamplingRequirements:
    requires_trajectory: bool = True
    requires_log_prob: bool = True
    requires_embeddings: bool = True
    requires_clean_latents: bool = False

    @property
    def is_forward_process(self) -> bool:
        return self.requires_clean_latents and not self.requires_trajectory

    def to_dict(self) -> Dict[str, bool]:
        return {k: bool(getattr(self, k)) for k in ("requires_trajectory", "requires_log_prob", "requires_embeddings")}


__all__ = ["BaseSamplingParams", "DiffusionSamplingParams", "ARSamplingParams", "ComposedSamplingParams",
           "SamplingRequirements", "get_diffusion_params", "get_ar_params"]
