"""``TrainStack`` — one rollout shard → ``num_updates_per_batch`` optimizer steps.

``train_track(track, training_progress)`` (``DP_SCATTER``): move the payload to the model device →
``prepare_segment`` (freeze π_old; replayed per micro-slice when the algorithm recomputes its anchor,
so old/new forwards share the exact batch geometry and the on-policy ratio is exactly 1) → for
each mini-batch: ``zero_grad``; per micro-slice ``set_grad_sync(last)`` +
``algorithm.compute_loss_and_backward(loss_scale = 1/n_micro)``; ``optimizer_step`` → ``on_rollout_end``.
Parity: ``unirl/train/stack.py:52-66`` (result), ``:75-108`` (slicing), ``:195-264`` (prepare), ``:266-344``
(train), ``:350-410`` (train_track).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Tuple

import torch

from unirl_b200.algorithms.base import AlgorithmStepResult, StageAlgorithm
from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.distributed.tensor.batch import _tree_apply
from unirl_b200.types.rollout_resp import RolloutTrack
from unirl_b200.utils.misc import aggregate_numeric_metrics

logger = logging.getLogger(__name__)


@dataclass(frozen=True)
class TrainStepResult:
    loss: float
    grad_norm: float
    lr: float
    has_backward: bool
    micros: List[AlgorithmStepResult]
    metrics: Mapping[str, object]
    per_update: Tuple[Mapping[str, object], ...] = ()


def _positive(name: str, v: Any) -> int:
    v = int(v)
    if v < 1:
        raise ValueError(f"{name} must be >= 1, got {v}")
    return v


def build_micro_batch_slices(*, total_size: int, micro_batch_size: int) -> Tuple[Tuple[int, int], ...]:
    n, m = _positive("total_size", total_size), _positive("micro_batch_size", micro_batch_size)
    return tuple((s, min(s + m, n)) for s in range(0, n, m))


def build_mini_batch_slices(*, total_size: int, num_updates: int) -> Tuple[Tuple[int, int], ...]:
    n, k = _positive("total_size", total_size), _positive("num_updates_per_batch", num_updates)
    if n % k:
        raise ValueError(f"num_updates_per_batch={k} must evenly divide the per-worker batch size ({n})")
    return tuple((i * (n // k), (i + 1) * (n // k)) for i in range(k))


def aggregate_update_results(results: List[TrainStepResult]) -> TrainStepResult:
    if len(results) == 1:
        return TrainStepResult(results[0].loss, results[0].grad_norm, results[0].lr, results[0].has_backward, results[0].micros,
                               results[0].metrics, (dict(results[0].metrics),))
    n = len(results)
    return TrainStepResult(sum(r.loss for r in results) / n, sum(r.grad_norm for r in results) / n, results[-1].lr,
                           any(r.has_backward for r in results), [m for r in results for m in r.micros],
                           aggregate_numeric_metrics([dict(r.metrics) for r in results if r.metrics]),
                           tuple(dict(r.metrics, loss=r.loss, grad_norm=r.grad_norm) for r in results))


def align_track_to_model(track: RolloutTrack, device: Any) -> None:
    """Segment, conditions and advantages to the model device; decoded media stays where it is."""
    if track.segment is not None:
        track.segment = track.segment.to_device(device)
    track.conditions = {k: _tree_apply(v, lambda t: t.to(device)) for k, v in track.conditions.items()}
    if track.advantages is not None:
        track.advantages = track.advantages.to(device)


class TrainStack(Remote):
    def __init__(self, *, fsdp_backend: Any, algorithm: StageAlgorithm, micro_batch_size: int, max_grad_norm: float,
                 num_updates_per_batch: int = 1) -> None:
        super().__init__()
        if int(micro_batch_size) < 1:
            raise ValueError(f"TrainStack.micro_batch_size must be >= 1, got {micro_batch_size}")
        if float(max_grad_norm) <= 0:
            raise ValueError(f"TrainStack.max_grad_norm must be > 0, got {max_grad_norm}")
        self.num_updates_per_batch = _positive("TrainStack.num_updates_per_batch", num_updates_per_batch)
        if self.num_updates_per_batch > 1 and not getattr(algorithm, "supports_multi_update", False):
            raise ValueError(f"num_updates_per_batch={self.num_updates_per_batch} needs an algorithm with a frozen π_old anchor; "
                             f"{type(algorithm).__name__} sets supports_multi_update=False")
        self.fsdp_backend, self.algorithm = fsdp_backend, algorithm
        self.micro_batch_size, self.max_grad_norm = int(micro_batch_size), float(max_grad_norm)

    def _optimizer_step_slices(self, total: int) -> List[List[Tuple[int, int]]]:
        """Per optimizer step, the absolute micro-batch ranges — shared by ``prepare_segment`` and ``train``."""
        return [[(lo + a, lo + b) for a, b in build_micro_batch_slices(total_size=hi - lo, micro_batch_size=self.micro_batch_size)]
                for lo, hi in build_mini_batch_slices(total_size=total, num_updates=self.num_updates_per_batch)]

    def prepare_segment(self, track: RolloutTrack) -> None:
        if track.segment is None:
            return
        algo = self.algorithm
        slices = [s for step in self._optimizer_step_slices(track.batch_size) for s in step]
        if not algo.recomputes_anchor() or len(slices) == 1:
            algo.prepare_segment(conditions=track.conditions, segment=track.segment)
            return
        parts: Dict[str, List[torch.Tensor]] = {f: [] for f in algo.anchor_fields}
        for lo, hi in slices:
            micro = track.slice(lo, hi)
            algo.prepare_segment(conditions=micro.conditions, segment=micro.segment)
            for f in parts:
                v = getattr(micro.segment, f, None)
                if v is None:
                    raise RuntimeError(f"{type(algo).__name__} declares anchor field {f!r} but a micro-slice produced None")
                parts[f].append(v)
        for f, vals in parts.items():
            setattr(track.segment, f, torch.cat(vals, 0))

    def train(self, track: RolloutTrack, *, micro_slices: List[Tuple[int, int]], training_progress: float) -> TrainStepResult:
        if track.advantages is None:
            raise ValueError("TrainStack.train: track.advantages is None")
        if not micro_slices:
            raise ValueError("TrainStack.train: empty micro_slices")
        be = self.fsdp_backend
        be.zero_grad()
        scale = 1.0 / len(micro_slices)
        whole = len(micro_slices) == 1 and micro_slices[0] == (0, track.batch_size)
        micros: List[AlgorithmStepResult] = []
        for i, (lo, hi) in enumerate(micro_slices):
            be.set_grad_sync(i == len(micro_slices) - 1)
            mt = track if whole else track.slice(lo, hi)
            micros.append(self.algorithm.compute_loss_and_backward(conditions=mt.conditions, segment=mt.segment, advantages=mt.advantages,
                                                                   training_progress=training_progress, loss_scale=scale))
        has_bwd = any(m.has_backward for m in micros)
        if hasattr(be, "any_rank"):
            has_bwd = be.any_rank(has_bwd)
        if has_bwd:
            grad_norm = float(be.optimizer_step(max_grad_norm=self.max_grad_norm))
        else:
            grad_norm = 0.0
            logger.warning("TrainStack.train: no micro-batch produced a backward; optimizer step skipped")
        return TrainStepResult(sum(m.loss for m in micros), grad_norm, float(be.current_lr), has_bwd, micros,
                               aggregate_numeric_metrics([m.metrics for m in micros if m.metrics]))

    def on_rollout_end(self) -> None:
        self.fsdp_backend.on_rollout_end()

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def train_track(self, resp_track: RolloutTrack, *, training_progress: float) -> TrainStepResult:
        dev = next(self.fsdp_backend.model.parameters()).device
        align_track_to_model(resp_track, dev)
        self.prepare_segment(resp_track)
        results = [self.train(resp_track, micro_slices=sl, training_progress=training_progress)
                   for sl in self._optimizer_step_slices(resp_track.batch_size)]
        self.on_rollout_end()
        out = aggregate_update_results(results)
        if torch.cuda.is_available():
            m = dict(out.metrics)
            m["cuda_max_allocated_gb"] = torch.cuda.max_memory_allocated() / 2**30
            out = TrainStepResult(out.loss, out.grad_norm, out.lr, out.has_backward, out.micros, m, out.per_update)
        return out


__all__ = ["TrainStack", "TrainStepResult", "build_micro_batch_slices", "build_mini_batch_slices", "aggregate_update_results", "align_track_to_model"]
