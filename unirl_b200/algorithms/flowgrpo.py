"""FlowGRPO — PPO clip on per-step Gaussian transition log-probs of a flow-matching sampler.

Also the loss behind the DanceGRPO and MixGRPO recipes (FlowGRPO + ``DanceSDEStrategy``, or +
``WindowScheduler`` choosing which steps are stochastic).  ``stage.replay(conditions, segment,
params, step_indices)`` returns ``log_probs [B, S']``; the anchor is ``segment.sde_logp`` — emitted by
the native sampler's fused SDE kernel (``old_logp_source="rollout"``) or recomputed without grad
at pre-update weights (``"replay"``).  Parity: ``unirl/algorithms/flowgrpo.py:44-206``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Type

import torch

from unirl_b200.algorithms.base import (
    AlgorithmStepResult,
    BaseAlgorithmConfig,
    StageAlgorithm,
    _resolve_stage,
    gather_sde_field,
    grpo_clip_loss,
    resolve_clip_range,
    typed_conditions,
)
from unirl_b200.config.require import require


@dataclass
class FlowGRPOConfig(BaseAlgorithmConfig):
    clip_range: float = 1e-4
    clip_schedule: str = "constant"
    old_logp_source: str = "rollout"


class FlowGRPO(StageAlgorithm):
    supports_multi_update = True
    anchor_fields = ("sde_logp",)

    def __init__(self, *, params: Any, stage: Any = None, pipeline: Any = None, stage_attr: str = "diffusion",
                 clip_range: float = 1e-4, clip_schedule: str = "constant", old_logp_source: str = "rollout",
                 conditions_cls: Optional[Type[Any]] = None) -> None:
        super().__init__()
        self.stage = _resolve_stage(stage, pipeline, stage_attr, type(self).__name__)
        self.params = params
        self.clip_range, self.clip_schedule = float(clip_range), str(clip_schedule)
        self.old_logp_source = str(old_logp_source).strip().lower()
        require(self.old_logp_source in ("rollout", "replay"), f"old_logp_source must be 'rollout' or 'replay', got {old_logp_source!r}")
        self.conditions_cls = conditions_cls

    def recomputes_anchor(self) -> bool:
        return self.old_logp_source == "replay"

    def _resolve_target_steps(self, segment: Any) -> List[int]:
        return [] if segment.sde_indices is None else [int(i) for i in segment.sde_indices.tolist()]

    def _replay(self, conditions: Mapping[str, Any], segment: Any, steps: List[int]) -> Any:
        return self.stage.replay(typed_conditions(conditions, self.conditions_cls), segment=segment, params=self.params, step_indices=steps)

    def prepare_segment(self, *, conditions: Mapping[str, Any], segment: Any) -> None:
        steps = self._resolve_target_steps(segment)
        if not steps:
            return
        if self.old_logp_source == "rollout":
            if segment.sde_logp is None:
                raise RuntimeError(f"{type(self).__name__}: old_logp_source='rollout' but the engine emitted no sde_logp; "
                                   "use old_logp_source='replay'")
            return
        with torch.no_grad():
            out = self._replay(conditions, segment, steps)
        segment.sde_logp = out.log_probs.detach()

    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult:
        steps = self._resolve_target_steps(segment)
        if not steps:
            return AlgorithmStepResult.skipped()
        new_logp = self._replay(conditions, segment, steps).log_probs
        old_logp = gather_sde_field(segment.sde_logp, segment.sde_indices, steps, field_name="sde_logp").to(new_logp)
        eps = resolve_clip_range(self.clip_range, self.clip_schedule, training_progress)
        adv = advantages.detach().to(new_logp).reshape(-1, 1).expand_as(new_logp)
        loss_elem, stats = grpo_clip_loss(new_logp=new_logp, old_logp=old_logp, advantages=adv, clip_range=eps)
        loss = loss_elem.mean()
        (loss * loss_scale).backward()
        metrics: Dict[str, Any] = {"policy_loss": float(loss.detach()), "clip_range": float(eps), **{k: float(v) for k, v in stats.items()}}
        return AlgorithmStepResult(float(loss.detach()), metrics, len(steps), True)


__all__ = ["FlowGRPO", "FlowGRPOConfig"]
