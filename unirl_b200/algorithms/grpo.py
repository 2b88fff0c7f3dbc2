"""GRPO over packed AR token segments.

``new_logp = stage.replay(conditions, segment, temperature=T)`` (``[total_tokens]``, fused
lm_head + log-softmax + gather on CUDA), anchor = rollout log-probs, per-sample advantages
broadcast over each sample's tokens, PPO clip with optional DAPO clip-higher, three aggregation
modes.  Parity: ``unirl/algorithms/grpo.py:40-199``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Type

import torch

from unirl_b200.algorithms.base import (
    AlgorithmStepResult,
    BaseAlgorithmConfig,
    StageAlgorithm,
    _resolve_stage,
    aggregate_token_loss,
    default_temperature,
    expand_per_token,
    grpo_clip_loss,
    resolve_clip_range,
    rollout_replay_logp_absdiff,
    typed_conditions,
)


@dataclass
class GRPOConfig(BaseAlgorithmConfig):
    clip_range: float = 1e-4
    clip_range_high: Optional[float] = None
    clip_schedule: str = "constant"
    loss_agg_mode: str = "token-mean"
    horizon: int = 8192


class GRPO(StageAlgorithm):
    supports_multi_update = True

    def __init__(self, *, stage: Any = None, pipeline: Any = None, stage_attr: str = "ar", clip_range: float = 1e-4,
                 clip_schedule: str = "constant", clip_range_high: Optional[float] = None, loss_agg_mode: str = "token-mean",
                 horizon: int = 8192, conditions_cls: Optional[Type[Any]] = None, sampling_temperature: Optional[float] = None) -> None:
        super().__init__()
        self.stage = _resolve_stage(stage, pipeline, stage_attr, "GRPO")
        self.clip_range = float(clip_range)
        self.clip_range_high = None if clip_range_high is None else float(clip_range_high)
        self.clip_schedule, self.loss_agg_mode, self.horizon = str(clip_schedule), str(loss_agg_mode), int(horizon)
        self.conditions_cls = conditions_cls
        self.sampling_temperature = default_temperature() if sampling_temperature is None else float(sampling_temperature)

    _expand_advantages_to_tokens = staticmethod(expand_per_token)

    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult:
        if segment.tokens is None or segment.lengths is None or segment.log_probs is None or not segment.tokens.shape[0]:
            return AlgorithmStepResult.skipped()
        new_logp = self.stage.replay(typed_conditions(conditions, self.conditions_cls), segment=segment, temperature=self.sampling_temperature)
        old_logp = segment.log_probs.to(dtype=new_logp.dtype, device=new_logp.device)
        adv = expand_per_token(advantages, segment.lengths, dtype=new_logp.dtype, device=new_logp.device)
        eps = resolve_clip_range(self.clip_range, self.clip_schedule, training_progress)
        eps_hi = None if self.clip_range_high is None else resolve_clip_range(self.clip_range_high, self.clip_schedule, training_progress)
        loss_elem, stats = grpo_clip_loss(new_logp=new_logp, old_logp=old_logp, advantages=adv, clip_range=eps, clip_range_high=eps_hi)
        if segment.loss_mask is not None:
            loss_elem = loss_elem * segment.loss_mask.to(loss_elem)
        loss = aggregate_token_loss(loss_elem, segment.lengths, self.loss_agg_mode, self.horizon)
        (loss * loss_scale).backward()
        metrics: Dict[str, Any] = {"policy_loss": float(loss.detach()), "clip_range": float(eps),
                                   **rollout_replay_logp_absdiff(new_logp, old_logp), **{k: float(v) for k, v in stats.items()}}
        return AlgorithmStepResult(float(loss.detach()), metrics, int(new_logp.shape[0]), True)


__all__ = ["GRPO", "GRPOConfig"]
