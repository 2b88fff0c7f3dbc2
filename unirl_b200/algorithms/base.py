"""Algorithm contract: an algorithm is a *loss node* that owns a stage and runs backward.

``StageAlgorithm.compute_loss_and_backward(conditions, segment, advantages, training_progress,
loss_scale)`` replays the segment through its stage (``ARStage.replay`` / ``DiffusionStage.replay``),
applies the policy-ratio loss and calls ``backward``; the train stack owns batching and the
optimizer.  The element-wise ratio/clip/penalty math lives in ``unirl_b200.ops.policy_loss`` — one
fused sm_100a kernel per loss family on CUDA, a PyTorch fp32 expression elsewhere.

Parity: ``unirl/algorithms/base.py:31-157`` (helpers), ``:182-298`` (contract).
"""

from __future__ import annotations

import math
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple, Type

import torch

from unirl_b200.distributed.group.remote import Remote
from unirl_b200.ops import policy_loss as PL


def typed_conditions(conditions: Mapping[str, Any], conditions_cls: Optional[Type[Any]]) -> Any:
    """Rebuild the stage's typed conditions container (``None`` ⇒ pass the dict through)."""
    if conditions_cls is None:
        return conditions
    if isinstance(conditions, conditions_cls):
        return conditions
    return conditions_cls.from_dict(dict(conditions))


def gather_sde_field(tensor: Optional[torch.Tensor], sde_indices: Optional[torch.Tensor], target_steps: List[int], *,
                     field_name: str = "field") -> torch.Tensor:
    """``tensor[:, slot(step) for step in target_steps]`` where ``slot`` inverts ``sde_indices``."""
    if tensor is None or sde_indices is None:
        raise ValueError(f"gather_sde_field: {field_name} or sde_indices missing (did prepare_segment run?)")
    slot = {int(s): k for k, s in enumerate(sde_indices.tolist())}
    missing = [t for t in target_steps if int(t) not in slot]
    if missing:
        raise ValueError(f"gather_sde_field({field_name}): steps {missing} not in sde_indices={sde_indices.tolist()}")
    return tensor[:, [slot[int(t)] for t in target_steps]]


def rollout_replay_logp_absdiff(new_logp: torch.Tensor, old_logp: torch.Tensor) -> Dict[str, float]:
    """|Δ log p| between the rollout engine and the teacher-forced replay: the engine-gap gauge."""
    with torch.no_grad():
        d = (new_logp - old_logp).abs()
    return {"rollout_replay_logp_absdiff_mean": float(d.mean()), "rollout_replay_logp_absdiff_max": float(d.max())}


def resolve_clip_range(clip_range: float, schedule: str, progress: float) -> float:
    if schedule == "linear_decay":
        return clip_range * (1.0 - 0.5 * float(progress))
    if schedule == "cosine_decay":
        return clip_range * 0.5 * (1.0 + math.cos(math.pi * float(progress)))
    return clip_range


_resolve_clip_range_from_schedule = resolve_clip_range


def grpo_clip_loss(*, new_logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, clip_range: float,
                   clip_range_high: Optional[float] = None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """PPO clip: ``max(−A·r, −A·clamp(r, 1−ε⁻, 1+ε⁺))`` element-wise + detached ratio statistics."""
    return PL.ppo_clip(new_logp, old_logp, advantages, clip_range, clip_range if clip_range_high is None else clip_range_high)


_grpo_clip_loss = grpo_clip_loss


def expand_per_token(values: torch.Tensor, lengths: torch.Tensor, *, dtype: torch.dtype, device: Any) -> torch.Tensor:
    if values.shape[0] != lengths.shape[0]:
        raise ValueError(f"advantage expansion: {values.shape[0]} samples vs {lengths.shape[0]} lengths")
    return torch.repeat_interleave(values.detach().to(device=device, dtype=dtype), lengths.to(device), dim=0)


def aggregate_token_loss(loss_elem: torch.Tensor, lengths: torch.Tensor, mode: str, horizon: int) -> torch.Tensor:
    """``token-mean`` | ``seq-mean-token-sum-norm`` (÷ horizon) | ``seq-mean-token-mean`` over packed tokens."""
    if mode == "token-mean":
        return loss_elem.mean()
    n = lengths.numel()
    seq_id = torch.repeat_interleave(torch.arange(n, device=loss_elem.device), lengths.to(loss_elem.device))
    sums = torch.zeros(n, dtype=loss_elem.dtype, device=loss_elem.device).index_add_(0, seq_id, loss_elem)
    if mode == "seq-mean-token-sum-norm":
        return sums.mean() / float(horizon)
    if mode == "seq-mean-token-mean":
        return (sums / lengths.to(sums).clamp(min=1)).mean()
    raise ValueError(f"unknown loss_agg_mode {mode!r}")


@dataclass(frozen=True)
class AlgorithmStepResult:
    loss: float
    metrics: Mapping[str, Any]
    num_steps_or_tokens: int
    has_backward: bool

    @classmethod
    def skipped(cls) -> "AlgorithmStepResult":
        return cls(0.0, {}, 0, False)


class BaseAlgorithmConfig(ABC):
    """Marker base for algorithm config dataclasses."""


class StageAlgorithm(Remote, ABC):
    """See module docstring.

    ``requires_ema_rollout``: sample with EMA weights (off-policy / forward-process methods).
    ``supports_multi_update``: correct under several optimizer steps per rollout (needs a frozen π_old).
    ``anchor_fields``: segment fields ``prepare_segment`` fills when it recomputes the anchor.
    """

    requires_ema_rollout: bool = False
    supports_multi_update: bool = False
    anchor_fields: Tuple[str, ...] = ()

    def recomputes_anchor(self) -> bool:
        """True ⇒ the anchor must be replayed at the exact micro-batch geometry training uses."""
        return False

    def prepare_segment(self, *, conditions: Mapping[str, Any], segment: Any) -> None:
        return None

    @abstractmethod
    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult: ...


def _resolve_stage(stage: Any, pipeline: Any, stage_attr: str, who: str) -> Any:
    if stage is None and pipeline is None:
        raise ValueError(f"{who}: pass `stage` or `pipeline`")
    return stage if stage is not None else getattr(pipeline, stage_attr)


def default_temperature() -> float:
    from unirl_b200.types.sampling import ARSamplingParams

    return float(ARSamplingParams.__dataclass_fields__["temperature"].default)


__all__ = ["AlgorithmStepResult", "StageAlgorithm", "BaseAlgorithmConfig", "typed_conditions", "gather_sde_field",
           "rollout_replay_logp_absdiff", "resolve_clip_range", "grpo_clip_loss", "expand_per_token", "aggregate_token_loss"]
