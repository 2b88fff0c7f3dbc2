"""``ARTrainer`` — GRPO / DRPO for autoregressive policies.

One step: (weight sync) → ``rollout.generate`` → ``reward.score_and_attach`` → group advantages on the
controller → (colocated: ``rollout.sleep``) → ``stack.train_track`` → metrics.  Roles are created from
recipe nodes inside placement scopes: *colocated* (default — every role on every device; trainer
and engine share each GPU) or *separate* (``rollout_fraction`` of the pool for the engine, the rest for
training, weights crossing slabs by broadcast or the fused reshard path).
Parity: ``unirl/trainer/ar.py:37-99`` (construction), ``:101-118`` (request), ``:120-171`` (step), ``:173-221`` (eval),
``:223-284`` (loop with resume fast-forward and forced first sync).
"""

from __future__ import annotations

import dataclasses
import inspect
import logging
import time
from typing import Any, Dict, Optional, Tuple

import torch

from unirl_b200.config.instantiate import instantiate, parse_cfg
from unirl_b200.distributed.group.placement import placement, remote, remote_cfg
from unirl_b200.trainer.base import BaseTrainer
from unirl_b200.types.prompts import RolloutInputs
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import hydrate_if_handle

logger = logging.getLogger(__name__)


class ARTrainer(BaseTrainer):
    def __init__(self, *, cfg: Any, batch_size: int, bundle_cfg: Any, pipeline_cfg: Any, backend_cfg: Any, rollout_cfg: Any, reward_cfg: Any,
                 algorithm_cfg: Any, stack_cfg: Any, data_source_cfg: Any, sampling_cfg: Any, sync_cfg: Any = None, logging_cfg: Any = None,
                 adv_normalization_scope: str = "group", normalize_adv_by_std: bool = True, eval_interval: int = 0, eval_num_prompts: int = 60,
                 eval_samples_per_prompt: int = 16, eval_temperature: float = 1.0, pool: Any = None) -> None:
        super().__init__(cfg=cfg, logging_cfg=logging_cfg, pool=pool)
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        self.batch_size = int(batch_size)
        self.adv_normalization_scope, self.normalize_adv_by_std = adv_normalization_scope, bool(normalize_adv_by_std)
        self.eval_interval, self.eval_num_prompts = int(eval_interval), int(eval_num_prompts)
        self.eval_samples_per_prompt, self.eval_temperature = int(eval_samples_per_prompt), float(eval_temperature)
        self.data_source = instantiate(data_source_cfg)
        self.sampling_params = instantiate(sampling_cfg)
        self.weight_sync = None
        # ``placement`` / ``rollout_fraction``; recipes written for the reference say ``layout`` and give the TRAINER's share (``train_fraction``)
        self.separate = str(get("placement", get("layout", "colocated"))) == "separate"
        rollout_fraction = float(get("rollout_fraction", 1.0 - float(get("train_fraction", 0.5))))
        rollout_parallel = get("rollout_parallel")
        rollout_parallel = dict(rollout_parallel) if rollout_parallel else None
        train_parallel = get("train_parallel")
        self._train_parallel = dict(train_parallel) if train_parallel else None  # e.g. {sp: 8}: sequence-parallel peers share every batch shard
        rp = parse_cfg(rollout_cfg)
        wants_pipeline = "pipeline" in inspect.signature(rp["role_cls"]).parameters
        wants_bundle = "bundle" in inspect.signature(rp["role_cls"]).parameters
        if not self.separate:
            with placement(self.pool, fraction=1.0, shared_workers=True):
                self._build_train_roles(bundle_cfg, pipeline_cfg, backend_cfg, algorithm_cfg, stack_cfg)
                extra: Dict[str, Any] = {}
                if wants_pipeline:
                    extra["pipeline"] = self.pipeline
                elif wants_bundle:
                    extra["bundle"] = self.bundle
                self.rollout = remote(**rp, parallel=rollout_parallel if rollout_parallel is not None else (self._train_parallel if wants_pipeline else None), **extra)
                self.reward = remote_cfg(reward_cfg)
                if sync_cfg is not None:
                    self.weight_sync = remote_cfg(sync_cfg, backend=self.backend, rollout=self.rollout)
        else:
            n_roll = max(1, int(round(self.pool.num_devices * rollout_fraction)))
            if n_roll >= self.pool.num_devices:
                raise ValueError(f"a separate layout needs at least one device for each of trainer and engine: {self.pool.num_devices} device(s), {n_roll} for the engine")
            with placement(self.pool, num_devices=self.pool.num_devices - n_roll):
                self._build_train_roles(bundle_cfg, pipeline_cfg, backend_cfg, algorithm_cfg, stack_cfg)
                if sync_cfg is not None:
                    self.weight_sync = remote_cfg(sync_cfg, backend=self.backend)
            with placement(self.pool, num_devices=n_roll):
                self.rollout = remote(**rp, parallel=rollout_parallel)
                self.reward = remote_cfg(reward_cfg)
            # across two device slabs: full weights travel by broadcast over a group of trainer rank 0 + engine ranks; LoRA adapters are
            # small and go through the controller (extract on the trainer, set_lora_from_tensors on every engine rank)
            self._sync_is_lora = self.weight_sync is not None and hasattr(getattr(self.weight_sync, "cls", None), "push")
            if self.weight_sync is not None and not self._sync_is_lora:
                from unirl_b200.distributed.weight_sync.driver import connect_nccl_sync

                connect_nccl_sync(self.weight_sync, self.rollout)
        self.last_sync_stats: Dict[str, float] = {}

    def _build_train_roles(self, bundle_cfg: Any, pipeline_cfg: Any, backend_cfg: Any, algorithm_cfg: Any, stack_cfg: Any) -> None:
        par = {"parallel": self._train_parallel} if self._train_parallel else {}
        self.bundle = remote_cfg(bundle_cfg, **par)
        self.pipeline = remote_cfg(pipeline_cfg, bundle=self.bundle, **par)
        self.backend = remote_cfg(backend_cfg, bundle=self.bundle, **par)
        algo_params = inspect.signature(parse_cfg(algorithm_cfg)["role_cls"]).parameters
        extra = {"backend": self.backend} if "backend" in algo_params else {}  # e.g. DiffusionNFT reads the EMA adapter policy from it
        self.algorithm = remote_cfg(algorithm_cfg, pipeline=self.pipeline, **extra, **par)
        self.stack = remote_cfg(stack_cfg, fsdp_backend=self.backend, algorithm=self.algorithm, **par)

    # ---- request ------------------------------------------------------------------------------------------
    def _build_req(self, inputs: RolloutInputs, rollout_id: int, sampling_params: Any = None) -> RolloutReq:
        sp = sampling_params or self.sampling_params
        inputs = inputs.expand(sp.samples_per_prompt)
        prims = dict(inputs.primitives)
        conds = {}
        if "prompt_tokens" in prims:
            conds["prompt"] = prims.pop("prompt_tokens")
        return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=prims, request_conditions=conds,
                          sampling_params=sp, metadata=list(inputs.metadata) if inputs.metadata else [])

    def _sync_weights(self) -> Dict[str, float]:
        if self.weight_sync is None:
            return {}
        if self.separate and getattr(self, "_sync_is_lora", False):
            from unirl_b200.distributed.weight_sync.lora.remote import sync_remote_lora

            stats = sync_remote_lora(self.weight_sync, self.rollout)
        elif self.separate:
            from unirl_b200.distributed.weight_sync.driver import drive_nccl_sync

            stats = drive_nccl_sync(self.weight_sync, self.rollout)
        else:
            per_rank = self.weight_sync.sync()
            stats = {k: max(float(r.get(k, 0.0)) for r in per_rank) for k in per_rank[0]} if per_rank else {}
        self.last_sync_stats = stats
        return stats

    # ---- one step --------------------------------------------------------------------------------------------
    def train_step(self, req: RolloutReq, *, training_progress: float = 0.0, sync_weights: bool = False, rollout_id: int = 0) -> Tuple[Any, float]:
        t0 = time.perf_counter()
        self.rollout.wake_up()
        sync_stats = self._sync_weights() if sync_weights else {}
        resp = self.rollout.generate(req)
        self.rollout.sleep()
        for name, track in list(resp.tracks.items()):
            if track.segment is not None:
                resp.tracks[name] = self.reward.score_and_attach(req=req, track=track)
        mean_reward = 0.0
        for name, track in list(resp.tracks.items()):
            if track.rewards is None:
                continue
            track.rewards = hydrate_if_handle(track.rewards)
            if isinstance(track.component_rewards, dict):
                track.component_rewards = {k: hydrate_if_handle(v) for k, v in track.component_rewards.items()}
            mean_reward = float(track.rewards.float().mean())
            resp.tracks[name] = track.compute_advantages(normalize=self.normalize_adv_by_std, scope=self.adv_normalization_scope)
        self._drop_decoded(req, resp, rollout_id=rollout_id)
        (track,) = resp.tracks.values()
        result = self.stack.train_track(track, training_progress=float(training_progress))
        lens = getattr(track.segment, "lengths", None) if track.segment is not None else None
        light = resp.metadata_only()
        if lens is not None:
            for t in light.tracks.values():
                t.segment = type(track.segment)()  # lengths only, for logging
                t.segment._set_cu(track.segment.cu_seqlens)
        self.wandb_logger.log_rollout_step(rollout_id, result, light, step_time_s=time.perf_counter() - t0,
                                           trunc_len=getattr(self.sampling_params, "max_new_tokens", None),
                                           timings=None, sync_stats=sync_stats, device_ms=dict(self.phase_timer.device_ms),
                                           roofline=self._roofline_info(req))
        return result, mean_reward

    def _roofline_info(self, req: Any) -> Optional[Dict[str, Any]]:
        """Static inputs of the per-step roofline metrics, when the bundle lives in this process (inline / spmd pools)."""
        info = getattr(self, "_roofline_static", None)
        if info is None:
            info = {}
            try:
                bundle = self.pool.local_role(self.bundle) if hasattr(self.pool, "local_role") else None
                model = getattr(bundle, "transformer", None)
                if model is not None:
                    cfg = model.cfg
                    n = sum(p.numel() for name, p in model.named_parameters() if not name.startswith("embed_tokens"))
                    info = {"n_params": n, "kv_bytes_per_token": 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2}
            except Exception:  # noqa: BLE001 - metrics only
                info = {}
            self._roofline_static = info
        if not info:
            return None
        out = dict(info)
        try:
            pt = req.primitives.get("prompt_tokens") if hasattr(req, "primitives") else None
            mask = getattr(pt, "attention_mask", None)
            if mask is not None:
                out["prompt_len_mean"] = float(mask.float().sum(-1).mean())
        except Exception:  # noqa: BLE001
            pass
        world = max(1, int(getattr(self, "num_devices", 1)))
        out["decode_batch"] = max(1, len(getattr(req, "sample_ids", [])) // world)
        return out

    def evaluate(self, rollout_id: int) -> float:
        inputs = self.data_source.get_eval_samples(self.eval_num_prompts)
        sp = dataclasses.replace(self.sampling_params, samples_per_prompt=self.eval_samples_per_prompt, temperature=self.eval_temperature)
        req = self._build_req(inputs, rollout_id, sp)
        self.rollout.wake_up()
        self._sync_weights()
        resp = self.rollout.generate(req)
        self.rollout.sleep()
        acc = 0.0
        for track in resp.tracks.values():
            if track.segment is not None:
                track = self.reward.score_and_attach(req=req, track=track)
            if track.rewards is not None:
                acc = float(hydrate_if_handle(track.rewards).float().mean())
                break
        logger.info("EVAL rollout %d  avg@%d over %d prompts = %.4f", rollout_id + 1, self.eval_samples_per_prompt, self.eval_num_prompts, acc)
        self.wandb_logger.log_eval(rollout_id + 1, {"acc": acc})
        return acc

    def train(self, *, num_rollouts: int, weight_sync_interval: int = 1, save_interval: int = 0, save_dir: Optional[str] = None,
              load_dir: Optional[str] = None, save_mode: str = "full") -> None:
        interval = max(1, weight_sync_interval)
        start = self.maybe_load_checkpoint(load_dir, num_rollouts=num_rollouts)
        resumed = bool(load_dir)
        for _ in range(start):  # fast-forward the data stream
            self.data_source.get_samples(self.batch_size)
        self._init_wandb(num_rollouts=num_rollouts, extra={"adv_normalization_scope": self.adv_normalization_scope})
        try:
            if self.eval_interval > 0:
                self.evaluate(rollout_id=-1)
            for rid in range(start, num_rollouts):
                progress = rid / max(1, num_rollouts - 1)
                req = self._build_req(self.data_source.get_samples(self.batch_size), rid)
                sync = (rid > 0 and rid % interval == 0) or (resumed and rid == start) or (self.separate and rid == 0)
                result, mean_reward = self.train_step(req, training_progress=progress, sync_weights=sync, rollout_id=rid)
                self.wandb_logger.log_progress(rid, num_rollouts, result, mean_reward, logger=logger)
                if self.eval_interval > 0 and (rid + 1) % self.eval_interval == 0:
                    self.evaluate(rollout_id=rid)
                self.maybe_save_checkpoint(rid, num_rollouts, save_interval=save_interval, save_dir=save_dir, save_mode=save_mode)
        finally:
            self._finish_wandb()


__all__ = ["ARTrainer"]
