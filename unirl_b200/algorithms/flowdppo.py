"""Flow-DPPO — divergence-masked policy optimisation for flow-matching samplers.

Instead of clipping the ratio, a transition is dropped from the loss when the KL between the new
and old Gaussian transition (shared variance ⇒ ``mean_{C,H,W}[(μ_new−μ_old)² / (2σ_t²)]``) reaches a
threshold *and* the ratio already moved in the advantage's direction:

    keep = not( kl ≥ τ  and  ((r > 1 and A > 0) or (r < 1 and A < 0)) ),   loss = where(keep, −A·r, 0).mean()

with ``σ_t = sqrt(s / (1 − min(s, .99)))·η·sqrt(−dt)``.  The anchor (``sde_logp`` **and** ``sde_means``)
only exists through a replay, so it is always recomputed at the exact micro-batch geometry.
Parity: ``unirl/algorithms/flowdppo.py:43-138`` (loss), ``:146-368`` (class).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple, Type

import torch

from unirl_b200.algorithms.base import (
    AlgorithmStepResult,
    BaseAlgorithmConfig,
    StageAlgorithm,
    _resolve_stage,
    gather_sde_field,
    typed_conditions,
)
from unirl_b200.ops import policy_loss as PL


def flowdppo_kl_adv_loss(*, new_logp: torch.Tensor, old_logp: torch.Tensor, new_means: torch.Tensor, old_means: torch.Tensor,
                         advantages: torch.Tensor, sigma_t: torch.Tensor, kl_mask_threshold: float) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    return PL.flow_dppo(new_logp, old_logp, new_means, old_means, advantages, sigma_t, float(kl_mask_threshold))


_flowdppo_kl_adv_loss = flowdppo_kl_adv_loss


@dataclass
class FlowDPPOConfig(BaseAlgorithmConfig):
    kl_mask_threshold: float = 1e-5
    add_kl_coefficient: bool = True
    old_logp_source: str = "replay"


class FlowDPPO(StageAlgorithm):
    supports_multi_update = True
    anchor_fields = ("sde_logp", "sde_means")

    def __init__(self, *, params: Any, stage: Any = None, pipeline: Any = None, stage_attr: str = "diffusion",
                 kl_mask_threshold: float = 1e-5, add_kl_coefficient: bool = True, old_logp_source: str = "replay",
                 conditions_cls: Optional[Type[Any]] = None) -> None:
        super().__init__()
        self.stage = _resolve_stage(stage, pipeline, stage_attr, "FlowDPPO")
        self.params = params
        self.kl_mask_threshold = float(kl_mask_threshold)
        self.add_kl_coefficient = bool(add_kl_coefficient)
        self.old_logp_source = str(old_logp_source).strip().lower()
        if self.old_logp_source not in ("rollout", "replay"):
            raise ValueError(f"FlowDPPO: old_logp_source must be 'rollout' or 'replay', got {old_logp_source!r}")
        self.conditions_cls = conditions_cls

    def recomputes_anchor(self) -> bool:
        return True

    def _resolve_target_steps(self, segment: Any) -> List[int]:
        return [] if segment.sde_indices is None else [int(i) for i in segment.sde_indices.tolist()]

    def _replay(self, conditions: Mapping[str, Any], segment: Any, steps: List[int]) -> Any:
        return self.stage.replay(typed_conditions(conditions, self.conditions_cls), segment=segment, params=self.params, step_indices=steps)

    def prepare_segment(self, *, conditions: Mapping[str, Any], segment: Any) -> None:
        steps = self._resolve_target_steps(segment)
        if not steps:
            return
        if self.old_logp_source == "rollout" and segment.sde_logp is not None and segment.sde_means is not None:
            return  # the native sampler emitted both anchors
        with torch.no_grad():
            out = self._replay(conditions, segment, steps)
        if out.prev_sample_means is None:
            raise RuntimeError("FlowDPPO: stage.replay returned no prev_sample_means")
        segment.sde_logp = out.log_probs.detach()
        segment.sde_means = out.prev_sample_means.detach()

    def _compute_sigma_t(self, segment: Any, steps: List[int], device: Any, ndim: int = 5) -> torch.Tensor:
        tail = [1] * (ndim - 2)
        if not self.add_kl_coefficient:
            return torch.ones(1, len(steps), *tail, device=device)
        if segment.sigmas is None:
            raise ValueError("FlowDPPO(add_kl_coefficient=True) needs segment.sigmas")
        sig = segment.sigmas.to(device=device, dtype=torch.float32)
        idx = torch.tensor(steps, dtype=torch.long, device=device)
        s, s_next = sig[idx], sig[idx + 1]
        std = torch.sqrt(s / (1.0 - torch.clamp(s, max=0.99))) * float(self.params.eta)
        return (std * torch.sqrt(-(s_next - s))).reshape(1, -1, *tail)

    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult:
        steps = self._resolve_target_steps(segment)
        if not steps:
            return AlgorithmStepResult.skipped()
        out = self._replay(conditions, segment, steps)
        new_logp, new_means = out.log_probs, out.prev_sample_means
        if new_means is None:
            raise RuntimeError("FlowDPPO: stage.replay returned no prev_sample_means")
        old_logp = gather_sde_field(segment.sde_logp, segment.sde_indices, steps, field_name="sde_logp").to(new_logp)
        old_means = gather_sde_field(segment.sde_means, segment.sde_indices, steps, field_name="sde_means").to(new_means)
        sigma_t = self._compute_sigma_t(segment, steps, new_logp.device, new_means.dim())
        adv = advantages.detach().to(new_logp).reshape(-1, 1).expand_as(new_logp)
        loss_elem, stats = flowdppo_kl_adv_loss(new_logp=new_logp, old_logp=old_logp, new_means=new_means, old_means=old_means,
                                                advantages=adv, sigma_t=sigma_t, kl_mask_threshold=self.kl_mask_threshold)
        loss = loss_elem.mean()
        (loss * loss_scale).backward()
        metrics: Dict[str, Any] = {"policy_loss": float(loss.detach()), "kl_mask_threshold": self.kl_mask_threshold,
                                   **{k: float(v) for k, v in stats.items()}}
        return AlgorithmStepResult(float(loss.detach()), metrics, len(steps), True)


__all__ = ["FlowDPPO", "FlowDPPOConfig", "flowdppo_kl_adv_loss"]
