"""``RolloutReq`` — everything one rollout needs, authored on the controller.

The controller is authoritative for the σ schedule (``sigmas``), the initial noise recipe
(``init_noise_group_ids`` + ``init_noise_latent_shape`` + ``sampling_params.seed``) and the SDE
step set; engines consume these verbatim and echo σ back for verification.  Parity:
``unirl/types/rollout_req.py:65-157``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, shared_field
from unirl_b200.types.conditions.base import Condition
from unirl_b200.types.sampling import BaseSamplingParams


def _fan_out(parent_ids: List[str], prefix: str, branch: int):
    child = [f"{p}/{prefix}{j}" for p in parent_ids for j in range(branch)]
    parents = [p for p in parent_ids for _ in range(branch)]
    return child, parents


@dataclass
class RolloutReq(Batch):
    sample_ids: List[str] = concat_field(default_factory=list)
    group_ids: List[str] = concat_field(default_factory=list)
    primitives: Dict[str, Any] = concat_field(default_factory=dict)
    request_conditions: Dict[str, Condition] = concat_field(default_factory=dict)
    sampling_params: Optional[BaseSamplingParams] = shared_field(default=None)
    stage_config: Dict[str, Any] = shared_field(default_factory=dict)
    sigmas: Optional[torch.Tensor] = shared_field(default=None)
    metadata: List[Optional[Dict[str, Any]]] = concat_field(default_factory=list)
    init_noise_group_ids: List[str] = concat_field(default_factory=list)
    init_noise_latent_shape: Optional[List[int]] = shared_field(default=None)

    @property
    def batch_size(self) -> int:
        return len(self.sample_ids) if self.sample_ids else super().batch_size

    def make_root_track(self, track_name: str, branch: int,
                        decode_to_condition: Optional[Callable[["RolloutReq"], Dict[str, Condition]]] = None,
                        new_segment: Optional[Any] = None) -> Any:
        """First fan-out: ``x`` prompts → ``x·branch`` root-track samples in group-by-parent order."""
        from unirl_b200.types.rollout_resp import RolloutTrack

        if not self.sample_ids:
            raise ValueError("make_root_track: request has no sample_ids")
        if branch < 1:
            raise ValueError(f"make_root_track: branch must be >= 1, got {branch}")
        ids, parents = _fan_out(self.sample_ids, track_name[:1] or "c", branch)
        conds = decode_to_condition(self) if decode_to_condition is not None else dict(self.request_conditions)
        return RolloutTrack(sample_ids=ids, parent_ids=parents, parent_track=None,
                            conditions={k: c.repeat_interleave(branch) for k, c in conds.items()}, segment=new_segment)


PrimitiveValue = Any

__all__ = ["RolloutReq", "PrimitiveValue"]
