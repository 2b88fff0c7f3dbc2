"""``UnifiedModelTrainStack`` — one sharded backend, two algorithms (text track and image track) on the same weights.

Per optimizer step both tracks back-propagate into the same gradient buffers (micro-batch by micro-batch, gradient sync
enabled only on the very last backward of the step), then ONE clip + optimizer step is taken.  The text and image losses
are weighted by ``ar_loss_weight`` / ``image_loss_weight``.  Parity: ``unirl/train/unified_model_stack.py:42-211``.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional, Tuple

import torch

from unirl_b200.algorithms.base import AlgorithmStepResult, StageAlgorithm
from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.train.stack import TrainStepResult, align_track_to_model, build_micro_batch_slices
from unirl_b200.types.rollout_resp import RolloutTrack
from unirl_b200.utils.misc import aggregate_numeric_metrics

logger = logging.getLogger(__name__)


class UnifiedModelTrainStack(Remote):
    def __init__(self, *, fsdp_backend: Any, ar_algorithm: Optional[StageAlgorithm], image_algorithm: Optional[StageAlgorithm], ar_micro_batch_size: int = 4,
                 image_micro_batch_size: int = 4, max_grad_norm: float = 1.0, ar_loss_weight: float = 1.0, image_loss_weight: float = 1.0,
                 micro_batch_size: Optional[int] = None) -> None:
        """``micro_batch_size``: one size for both tracks (the reference's single knob); the per-track sizes apply when it is not given."""
        super().__init__()
        if micro_batch_size is not None:
            if int(micro_batch_size) < 1:
                raise ValueError(f"UnifiedModelTrainStack.micro_batch_size must be at least 1, got {micro_batch_size}")
            ar_micro_batch_size = image_micro_batch_size = int(micro_batch_size)
        if float(max_grad_norm) <= 0.0:
            raise ValueError(f"UnifiedModelTrainStack.max_grad_norm must be positive, got {max_grad_norm}")
        self.fsdp_backend = fsdp_backend
        self.algorithms = {"ar": ar_algorithm, "image": image_algorithm}
        self.micro = {"ar": int(ar_micro_batch_size), "image": int(image_micro_batch_size)}
        self.weights = {"ar": float(ar_loss_weight), "image": float(image_loss_weight)}
        self.max_grad_norm = float(max_grad_norm)

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def train_tracks(self, ar_track: Optional[RolloutTrack] = None, image_track: Optional[RolloutTrack] = None, *, training_progress: float = 0.0) -> TrainStepResult:
        be = self.fsdp_backend
        dev = next(be.model.parameters()).device
        work: List[Tuple[str, RolloutTrack, Tuple[int, int], float]] = []
        for name, track in (("ar", ar_track), ("image", image_track)):
            algo = self.algorithms[name]
            if track is None or algo is None or track.segment is None:
                continue
            if track.advantages is None:
                raise ValueError(f"UnifiedModelTrainStack: track {name!r} has no advantages")
            align_track_to_model(track, dev)
            algo.prepare_segment(conditions=track.conditions, segment=track.segment)
            slices = build_micro_batch_slices(total_size=track.batch_size, micro_batch_size=self.micro[name])
            work += [(name, track, s, self.weights[name] / len(slices)) for s in slices]
        if not work:
            raise ValueError("UnifiedModelTrainStack.train_tracks: nothing to train on")
        be.zero_grad()
        micros: List[AlgorithmStepResult] = []
        metrics: List[Dict[str, Any]] = []
        for i, (name, track, (lo, hi), scale) in enumerate(work):
            be.set_grad_sync(i == len(work) - 1)
            mt = track if (lo, hi) == (0, track.batch_size) else track.slice(lo, hi)
            r = self.algorithms[name].compute_loss_and_backward(conditions=mt.conditions, segment=mt.segment, advantages=mt.advantages,
                                                                 training_progress=training_progress, loss_scale=scale)
            micros.append(r)
            if r.metrics:
                metrics.append({f"{name}/{k}": v for k, v in r.metrics.items()})
        has_bwd = any(m.has_backward for m in micros)
        if hasattr(be, "any_rank"):
            has_bwd = be.any_rank(has_bwd)
        grad_norm = float(be.optimizer_step(max_grad_norm=self.max_grad_norm)) if has_bwd else 0.0
        be.on_rollout_end()
        return TrainStepResult(sum(m.loss for m in micros), grad_norm, float(be.current_lr), has_bwd, micros, aggregate_numeric_metrics(metrics))


__all__ = ["UnifiedModelTrainStack"]
