"""DRPO — divergence-regularised policy optimisation for token-level policies.

Per token ``L = −A·r + |A|·μ·(r−1)² / (2ε)`` with ``r = π/μ`` kept differentiable, ``μ = exp(old_logp)``
the rollout-policy token probability (``penalty_mu_weighted=False`` drops the μ weight ⇒ plain SPO),
``log r`` clamped to ±20.  ``old_logp_source="replay"`` re-anchors on a no-grad replay at pre-update
weights.  Parity: ``unirl/algorithms/drpo.py:97-159`` (loss), ``:167-344`` (class).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Type

import torch

from unirl_b200.algorithms.base import (
    AlgorithmStepResult,
    BaseAlgorithmConfig,
    StageAlgorithm,
    aggregate_token_loss,
    default_temperature,
    expand_per_token,
    rollout_replay_logp_absdiff,
    typed_conditions,
)
from unirl_b200.ops import policy_loss as PL


def drpo_loss(*, new_logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, epsilon: float,
              mu_weighted: bool = True) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    return PL.drpo(new_logp, old_logp, advantages, float(epsilon), bool(mu_weighted))


_drpo_loss = drpo_loss


@dataclass
class DRPOConfig(BaseAlgorithmConfig):
    drpo_epsilon: float = 12.5
    penalty_mu_weighted: bool = True
    loss_agg_mode: str = "token-mean"
    horizon: int = 8192
    old_logp_source: str = "rollout"


class DRPO(StageAlgorithm):
    supports_multi_update = True

    def __init__(self, *, pipeline: Any = None, stage: Any = None, stage_attr: str = "ar", drpo_epsilon: float = 12.5,
                 penalty_mu_weighted: bool = True, loss_agg_mode: str = "token-mean", horizon: int = 8192,
                 sampling_temperature: Optional[float] = None, old_logp_source: str = "rollout",
                 conditions_cls: Optional[Type[Any]] = None) -> None:
        super().__init__()
        if pipeline is None and stage is None:
            raise ValueError("DRPO: `pipeline` (or `stage`) must be provided")
        self.stage = stage if stage is not None else getattr(pipeline, stage_attr)
        self.drpo_epsilon, self.penalty_mu_weighted = float(drpo_epsilon), bool(penalty_mu_weighted)
        self.loss_agg_mode, self.horizon = str(loss_agg_mode), int(horizon)
        self.sampling_temperature = default_temperature() if sampling_temperature is None else float(sampling_temperature)
        self.conditions_cls = conditions_cls
        self.old_logp_source = str(old_logp_source).strip().lower()
        if self.old_logp_source not in ("rollout", "replay"):
            raise ValueError(f"DRPO: old_logp_source must be 'rollout' or 'replay', got {old_logp_source!r}")

    def prepare_segment(self, *, conditions: Mapping[str, Any], segment: Any) -> None:
        if self.old_logp_source != "replay" or segment.tokens is None or segment.log_probs is None or not segment.tokens.shape[0]:
            return
        with torch.no_grad():
            frozen = self.stage.replay(typed_conditions(conditions, self.conditions_cls), segment=segment, temperature=self.sampling_temperature)
        segment.log_probs = frozen.detach().to(segment.log_probs.device)

    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult:
        if segment.tokens is None or segment.lengths is None or segment.log_probs is None or not segment.tokens.shape[0]:
            return AlgorithmStepResult.skipped()
        new_logp = self.stage.replay(typed_conditions(conditions, self.conditions_cls), segment=segment, temperature=self.sampling_temperature)
        old_logp = segment.log_probs.to(dtype=new_logp.dtype, device=new_logp.device)
        adv = expand_per_token(advantages, segment.lengths, dtype=new_logp.dtype, device=new_logp.device)
        loss_elem, stats = drpo_loss(new_logp=new_logp, old_logp=old_logp, advantages=adv, epsilon=self.drpo_epsilon,
                                     mu_weighted=self.penalty_mu_weighted)
        if segment.loss_mask is not None:
            loss_elem = loss_elem * segment.loss_mask.to(loss_elem)
        mode = self.loss_agg_mode if self.loss_agg_mode == "seq-mean-token-sum-norm" else "token-mean"
        loss = aggregate_token_loss(loss_elem, segment.lengths, mode, self.horizon)
        (loss * loss_scale).backward()
        metrics: Dict[str, Any] = {"policy_loss": float(loss.detach()), "drpo_epsilon": self.drpo_epsilon,
                                   **rollout_replay_logp_absdiff(new_logp, old_logp), **{k: float(v) for k, v in stats.items()}}
        return AlgorithmStepResult(float(loss.detach()), metrics, int(new_logp.shape[0]), True)


__all__ = ["DRPO", "DRPOConfig", "drpo_loss"]
