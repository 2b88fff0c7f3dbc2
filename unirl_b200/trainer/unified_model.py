"""``UnifiedModelTrainer`` — RL for a unified text + image model: ONE set of trainable weights, two rollout roles.

The model both reasons about / rewrites the prompt (text track ``"ar"``) and renders the image (track ``"image"``).  One
sharded backend holds the weights; an AR rollout engine and an image rollout engine generate from them (train-side
engines share the trainer's module; engines with their own copy receive weights through the configured sync handlers —
``extract`` on the trainer, offload the optimizer, wake the engines, ``push``).  Images are scored, the text track inherits
its sample's image reward, both tracks get group-relative advantages and a single optimizer step is taken on the sum of
the two losses (:class:`UnifiedModelTrainStack`).  Optional rollout dump for offline inspection.
Parity: ``unirl/trainer/unified_model.py:86-127, 133-304, 331-497, 499-614, 616-750``.
"""

from __future__ import annotations

import inspect
import json
import logging
import os
import time
from typing import Any, Dict, Optional, Tuple

from unirl_b200.config.instantiate import instantiate, parse_cfg
from unirl_b200.distributed.group.placement import placement, remote, remote_cfg
from unirl_b200.trainer.base import BaseTrainer
from unirl_b200.types.prompts import RolloutInputs
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import hydrate_if_handle
from unirl_b200.types.sampling import get_diffusion_params

logger = logging.getLogger(__name__)


class UnifiedModelTrainer(BaseTrainer):
    def __init__(self, *, cfg: Any, batch_size: int, bundle_cfg: Any, pipeline_cfg: Any, backend_cfg: Any, rollout_cfg: Any, reward_cfg: Any,
                 ar_algorithm_cfg: Any, image_algorithm_cfg: Any, stack_cfg: Any, data_source_cfg: Any, sampling_cfg: Any, sync_cfg: Any = None,
                 logging_cfg: Any = None, mode: str = "t2i", rollout_dump_dir: Optional[str] = None, adv_normalization_scope: str = "group",
                 normalize_adv_by_std: bool = True, pool: Any = None) -> None:
        super().__init__(cfg=cfg, logging_cfg=logging_cfg, pool=pool)
        self.batch_size, self.mode, self.rollout_dump_dir = int(batch_size), str(mode), rollout_dump_dir
        self.adv_normalization_scope, self.normalize_adv_by_std = adv_normalization_scope, bool(normalize_adv_by_std)
        self.data_source = instantiate(data_source_cfg)
        self.sampling_params = instantiate(sampling_cfg)
        with placement(self.pool, fraction=1.0, shared_workers=True):
            self.bundle = remote_cfg(bundle_cfg)
            self.pipeline = remote_cfg(pipeline_cfg, bundle=self.bundle)
            self.backend = remote_cfg(backend_cfg, bundle=self.bundle)
            self.ar_algorithm = remote_cfg(ar_algorithm_cfg, pipeline=self.pipeline) if ar_algorithm_cfg is not None else None
            self.image_algorithm = remote_cfg(image_algorithm_cfg, pipeline=self.pipeline) if image_algorithm_cfg is not None else None
            self.stack = remote_cfg(stack_cfg, fsdp_backend=self.backend, ar_algorithm=self.ar_algorithm, image_algorithm=self.image_algorithm)
            rp = parse_cfg(rollout_cfg)
            params = inspect.signature(rp["role_cls"]).parameters
            self.rollout = remote(**rp, **({"pipeline": self.pipeline} if "pipeline" in params else {}))
            self.reward = remote_cfg(reward_cfg)
            self.weight_sync = remote_cfg(sync_cfg, backend=self.backend, rollout=self.rollout) if sync_cfg is not None else None
        self._sched_shift = float(_get(bundle_cfg, "config.shift", 3.0))

    def _build_req(self, inputs: RolloutInputs, rollout_id: int) -> RolloutReq:
        sp = self.sampling_params
        d = get_diffusion_params(sp)
        inputs = inputs.expand(int(d.samples_per_prompt))
        gids = list(inputs.group_ids if d.init_same_noise else inputs.sample_ids)
        return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=dict(inputs.primitives), sampling_params=sp,
                          stage_config={"rollout_id": int(rollout_id), "mode": self.mode}, metadata=list(inputs.metadata) if inputs.metadata else [],
                          init_noise_group_ids=gids)

    def _dump(self, rollout_id: int, resp: Any) -> None:
        if not self.rollout_dump_dir:
            return
        os.makedirs(self.rollout_dump_dir, exist_ok=True)
        rows = []
        for name, t in resp.tracks.items():
            texts = getattr(t.decoded, "texts", None)
            for i, sid in enumerate(t.sample_ids):
                rows.append({"track": name, "sample_id": sid, "reward": None if t.rewards is None else float(t.rewards[i]),
                             "text": texts[i] if texts is not None else None})
        with open(os.path.join(self.rollout_dump_dir, f"rollout_{rollout_id:06d}.jsonl"), "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")

    def train_step(self, req: RolloutReq, *, training_progress: float = 0.0, sync_weights: bool = False, rollout_id: int = 0) -> Tuple[Any, float]:
        t0 = time.perf_counter()
        self.rollout.wake_up()
        if sync_weights and self.weight_sync is not None:
            self.weight_sync.sync()
        resp = self.rollout.generate(req)
        self.rollout.sleep()
        leaf = "image" if "image" in resp.tracks else "ar"
        resp.tracks[leaf] = self.reward.score_and_attach(req=req, track=resp.tracks[leaf])
        rewards = hydrate_if_handle(resp.tracks[leaf].rewards)
        resp.tracks[leaf].rewards = rewards
        if leaf == "image" and "ar" in resp.tracks:  # the rewrite is judged by the image it led to
            resp.tracks["ar"].rewards = rewards.clone()
        self._dump(rollout_id, resp)
        tracks = {}
        for name, t in resp.tracks.items():
            t = t.compute_advantages(normalize=self.normalize_adv_by_std, scope=self.adv_normalization_scope)
            t.decoded = None
            tracks[name] = resp.tracks[name] = t
        result = self.stack.train_tracks(tracks.get("ar"), tracks.get("image"), training_progress=float(training_progress))
        self.wandb_logger.log_rollout_step(rollout_id, result, resp.metadata_only(), step_time_s=time.perf_counter() - t0,
                                           device_ms=dict(self.phase_timer.device_ms))
        return result, float(rewards.float().mean())

    def train(self, *, num_rollouts: int, weight_sync_interval: int = 1, save_interval: int = 0, save_dir: Optional[str] = None,
              load_dir: Optional[str] = None, save_mode: str = "full") -> None:
        start = self.maybe_load_checkpoint(load_dir, num_rollouts=num_rollouts)
        for _ in range(start):
            self.data_source.get_samples(self.batch_size)
        self._init_wandb(num_rollouts=num_rollouts)
        try:
            for rid in range(start, num_rollouts):
                req = self._build_req(self.data_source.get_samples(self.batch_size), rid)
                result, mean_reward = self.train_step(req, training_progress=rid / max(1, num_rollouts - 1),
                                                      sync_weights=rid > 0 and rid % max(1, weight_sync_interval) == 0, rollout_id=rid)
                self.wandb_logger.log_progress(rid, num_rollouts, result, mean_reward, logger=logger)
                self.maybe_save_checkpoint(rid, num_rollouts, save_interval=save_interval, save_dir=save_dir, save_mode=save_mode)
        finally:
            self._finish_wandb()


def _get(node: Any, dotted: str, default: Any = None) -> Any:
    cur = node
    for part in dotted.split("."):
        if cur is None:
            return default
        cur = cur.get(part) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


__all__ = ["UnifiedModelTrainer"]
