"""In-process rollout on the trainer's own module(s): eval-scope, ``no_grad``, σ pinned on the request,
optional chunking by ``forward_batch_size``.  Because rollout and training share one module object
the "weight sync" of this engine is the identity.  Parity: ``unirl/rollout/engine/trainside/engine.py:28-125``.
"""

from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.rollout.engine.base import BaseRolloutEngine, chunked_engine_generate_req
from unirl_b200.sde.runtime import FlowMatchSchedulePolicy, ensure_req_sigmas
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp


class TrainsideRolloutEngine(BaseRolloutEngine):
    _component_name = "trainside"

    def __init__(self, *, pipeline: Any, stage: Optional[Any] = None, stage_attrs: Sequence[str] = ("diffusion",),
                 forward_batch_size: Optional[int] = None) -> None:
        super().__init__()
        self.pipeline = pipeline
        stages = [stage] if stage is not None else [getattr(pipeline, a) for a in stage_attrs]
        self._stages = stages
        self._models = [s.trainable_module() for s in stages]
        if forward_batch_size is not None and forward_batch_size < 1:
            raise ValueError(f"forward_batch_size must be >= 1 when set, got {forward_batch_size!r}")
        self.forward_batch_size = forward_batch_size
        self.schedule_policy: Optional[FlowMatchSchedulePolicy] = None
        if any(hasattr(s, "diffuse") for s in stages):
            if hasattr(pipeline, "build_schedule_policy"):
                self.schedule_policy = pipeline.build_schedule_policy()
            else:
                self.schedule_policy = FlowMatchSchedulePolicy.from_pretrained(getattr(pipeline.bundle, "pretrained_path", None),
                                                                               shift=float(getattr(pipeline, "shift", 3.0)))

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def generate(self, req: RolloutReq) -> RolloutResp:
        if self.schedule_policy is not None:
            ensure_req_sigmas(req, self.schedule_policy)
        modes = [m.training for m in self._models]
        for m in self._models:
            m.eval()
        try:
            with torch.no_grad():
                return chunked_engine_generate_req(req, self.pipeline.generate, self.forward_batch_size)
        finally:
            for m, mode in zip(self._models, modes):
                m.train(mode)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sleep(self) -> None:
        for s in self._stages:
            gen = getattr(s, "_gen", None)
            if gen is not None:
                gen.release_cache()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def wake_up(self) -> None:
        return None

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def health_check(self) -> bool:
        return self.pipeline is not None and all(m is not None for m in self._models)


__all__ = ["TrainsideRolloutEngine"]
