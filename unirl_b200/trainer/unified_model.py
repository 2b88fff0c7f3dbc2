"""``UnifiedModelTrainer`` — RL for a unified text + image model: ONE set of trainable weights, two rollout roles.

The model both reasons about / rewrites the prompt (text track ``"ar"``) and renders the image (track ``"image"``).  One
sharded backend holds the weights; an AR rollout engine and an image rollout engine generate from them (train-side
engines share the trainer's module; engines with their own copy receive weights through the configured sync handlers —
``extract`` on the trainer, offload the trainer, wake the engines, ``push``; see the class docstring for the two-engine mode).  Images are scored, the text track inherits
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
from typing import Any, Dict, List, Optional, Tuple

from unirl_b200.config.instantiate import instantiate, parse_cfg
from unirl_b200.distributed.group.placement import placement, remote, remote_cfg
from unirl_b200.trainer.base import BaseTrainer
from unirl_b200.types.primitives import Texts
from unirl_b200.types.prompts import RolloutInputs
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import hydrate_if_handle
from unirl_b200.types.sampling import get_diffusion_params

logger = logging.getLogger(__name__)


AR_TRACK, IMAGE_TRACK = "ar", "image"


class UnifiedModelTrainer(BaseTrainer):
    """Two ways to roll out:

    * ``rollout_cfg`` — ONE engine runs the whole text → image chain (train-side engine on the trainer's module).
    * ``ar_rollout_cfg`` + ``dit_rollout_cfg`` — an (AR, DiT) engine PAIR per replica, each engine on its own devices of the
      replica (first half / second half), with the memory choreography of a colocated large model:

          extract adapter / weights (trainer resident, engines asleep) → offload the trainer → wake the engines → push →
          rollout (P prompts → P·N rewrites on the AR engine → P·N·M images on the DiT engine) → engines asleep →
          trainer back on the device → score, credit assignment, advantages → two backward passes, one optimizer step → offload.

      Replicas (``devices_per_replica`` devices each) split the prompts of a step between them.
    """

    def __init__(self, *, cfg: Any, batch_size: int, bundle_cfg: Any, pipeline_cfg: Any, backend_cfg: Any, reward_cfg: Any,
                 ar_algorithm_cfg: Any, image_algorithm_cfg: Any, stack_cfg: Any, data_source_cfg: Any, sampling_cfg: Any, rollout_cfg: Any = None,
                 ar_rollout_cfg: Any = None, dit_rollout_cfg: Any = None, sync_cfg: Any = None, logging_cfg: Any = None, mode: str = "t2i",
                 rollout_dump_dir: Optional[str] = None, dump_dir: Optional[str] = None, adv_normalization_scope: str = "group",
                 normalize_adv_by_std: bool = True, enable_fsdp_offload: bool = False, devices_per_replica: Optional[int] = None,
                 pool: Any = None) -> None:
        super().__init__(cfg=cfg, logging_cfg=logging_cfg, pool=pool)
        self.batch_size, self.mode = int(batch_size), str(mode)
        self.rollout_dump_dir = rollout_dump_dir or dump_dir
        self.adv_normalization_scope, self.normalize_adv_by_std = adv_normalization_scope, bool(normalize_adv_by_std)
        self._enable_fsdp_offload = bool(enable_fsdp_offload)
        self.data_source = instantiate(data_source_cfg)
        self.sampling_params = instantiate(sampling_cfg)
        self.two_engines = ar_rollout_cfg is not None or dit_rollout_cfg is not None
        if self.two_engines and (ar_rollout_cfg is None or dit_rollout_cfg is None or rollout_cfg is not None):
            raise ValueError("UnifiedModelTrainer: give either rollout_cfg, or BOTH ar_rollout_cfg and dit_rollout_cfg")
        if not self.two_engines and rollout_cfg is None:
            raise ValueError("UnifiedModelTrainer: no rollout engine configured")
        self.weight_sync = None
        self.ar_rollouts: List[Any] = []
        self.dit_rollouts: List[Any] = []
        self._engine_syncs: List[Any] = []
        with placement(self.pool, fraction=1.0, shared_workers=True) as scope:
            self.bundle = remote_cfg(bundle_cfg)
            self.pipeline = remote_cfg(pipeline_cfg, bundle=self.bundle)
            self.backend = remote_cfg(backend_cfg, bundle=self.bundle)
            self.reward = remote_cfg(reward_cfg)
            self.ar_algorithm = remote_cfg(ar_algorithm_cfg, pipeline=self.pipeline) if ar_algorithm_cfg is not None else None
            self.image_algorithm = remote_cfg(image_algorithm_cfg, pipeline=self.pipeline) if image_algorithm_cfg is not None else None
            self.stack = remote_cfg(stack_cfg, fsdp_backend=self.backend, ar_algorithm=self.ar_algorithm, image_algorithm=self.image_algorithm)
            if not self.two_engines:
                self.rollout = self._wire_engine(rollout_cfg, list(scope.devices))
                self.weight_sync = remote_cfg(sync_cfg, backend=self.backend, rollout=self.rollout) if sync_cfg is not None else None
            else:
                # the engines of a colocated large model must find the trainer's state off the device when they come up
                if self._enable_fsdp_offload:
                    self.backend.offload()
                devs = list(scope.devices)
                per = int(devices_per_replica or len(devs))
                if per < 1 or len(devs) % per:
                    raise ValueError(f"UnifiedModelTrainer: {len(devs)} devices do not split into replicas of {per}")
                self.dp = len(devs) // per
                for r in range(self.dp):
                    mine = devs[r * per : (r + 1) * per]
                    half = max(1, per // 2)
                    ar_devs, dit_devs = (mine[:half], mine[half:]) if per >= 2 else (mine, mine)
                    # one engine at a time: build, let it finish coming up (the sleep call returns only then), put it to sleep
                    ar = self._wire_engine(ar_rollout_cfg, ar_devs)
                    ar.sleep()
                    self.ar_rollouts.append(ar)
                    dit = self._wire_engine(dit_rollout_cfg, dit_devs)
                    dit.sleep()
                    self.dit_rollouts.append(dit)
                self.rollout = self.ar_rollout = self.ar_rollouts[0]
                self.dit_rollout = self.dit_rollouts[0]
                if sync_cfg is not None:
                    sp = parse_cfg(sync_cfg)
                    params = inspect.signature(sp["role_cls"]).parameters
                    if hasattr(sp["role_cls"], "extract") and hasattr(sp["role_cls"], "push"):
                        # extract once on the trainer ranks, push the cached payload to every engine (cross-slab handler)
                        self.weight_sync = remote(**sp, backend=self.backend, **({"rollout": self.ar_rollouts[0]} if "rollout" in params else {}))
                    else:
                        self._engine_syncs = [remote(**dict(sp), backend=self.backend, rollout=eng) for eng in self.ar_rollouts + self.dit_rollouts]
        self._sched_shift = float(_get(bundle_cfg, "config.shift", 3.0))
        self._rollout_id = 0

    def _wire_engine(self, cfg: Any, devices: List[int]) -> Any:
        rp = parse_cfg(cfg)
        params = inspect.signature(rp["role_cls"]).parameters
        role_cls = rp.pop("role_cls")
        if "pipeline" in params:
            rp["pipeline"] = self.pipeline
        return self.pool.create_remote(role_cls, devices, **rp)

    # ---- requests ---------------------------------------------------------------------------------------------
    def _build_req(self, inputs: RolloutInputs, rollout_id: int) -> RolloutReq:
        sp = self.sampling_params
        d = get_diffusion_params(sp)
        if self.two_engines:
            # no pre-expansion: the rollout fans P prompts out to P·N rewrites and P·N·M images itself
            return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=dict(inputs.primitives), sampling_params=sp,
                              stage_config={"rollout_id": int(rollout_id), "mode": self.mode}, metadata=list(inputs.metadata) if inputs.metadata else [])
        inputs = inputs.expand(int(d.samples_per_prompt))
        gids = list(inputs.group_ids if d.init_same_noise else inputs.sample_ids)
        return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=dict(inputs.primitives), sampling_params=sp,
                          stage_config={"rollout_id": int(rollout_id), "mode": self.mode}, metadata=list(inputs.metadata) if inputs.metadata else [],
                          init_noise_group_ids=gids)

    # ---- two-engine rollout -----------------------------------------------------------------------------------
    def run_rollout(self, req: RolloutReq) -> Any:
        """Split the prompts over the replicas (contiguous, near-equal), run each part on its (AR, DiT) pair, concatenate the tracks."""
        from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack

        texts = req.primitives.get("text")
        n = len(texts.texts)
        if self.dp <= 1 or n <= 1:
            return self._run_rollout_one(self.ar_rollouts[0], self.dit_rollouts[0], req)
        bounds = [(n * r) // self.dp for r in range(self.dp + 1)]
        parts = []
        for r in range(self.dp):
            lo, hi = bounds[r], bounds[r + 1]
            if lo >= hi:
                continue
            sub = RolloutReq(sample_ids=list(req.sample_ids[lo:hi]), group_ids=list(req.group_ids[lo:hi]), primitives={"text": Texts(texts=list(texts.texts[lo:hi]))},
                             sampling_params=req.sampling_params, stage_config=dict(req.stage_config or {}),
                             metadata=list(req.metadata[lo:hi]) if req.metadata else [])
            parts.append(self._run_rollout_one(self.ar_rollouts[r], self.dit_rollouts[r], sub))
        return RolloutResp(tracks={name: RolloutTrack.concat([p.tracks[name] for p in parts]) for name in (AR_TRACK, IMAGE_TRACK)})

    def _run_rollout_one(self, ar_engine: Any, dit_engine: Any, req: RolloutReq) -> Any:
        """P prompts → (AR engine) P·N rewrites → (DiT engine) P·N·M images, with the lineage (sample ids, parents) built here and the
        engines' segments / conditions / decoded payloads grafted onto it.  Initial noise is requested per image and per ROLLOUT
        (``r<rollout>:<sample id>``), so the same prompt does not meet the same noise again in a later step."""
        from unirl_b200.types.rollout_resp import RolloutResp
        from unirl_b200.types.sampling import get_ar_params

        prompts = list(req.primitives["text"].texts)
        ar_params, diff_params = get_ar_params(req.sampling_params), get_diffusion_params(req.sampling_params)
        n_rec = int(ar_params.samples_per_prompt) if ar_params is not None else 1
        n_img = int(diff_params.samples_per_prompt)
        rid = int((req.stage_config or {}).get("rollout_id", self._rollout_id))
        ar_shell = req.make_root_track(track_name=AR_TRACK, branch=n_rec)
        ar_req = RolloutReq(sample_ids=list(ar_shell.sample_ids), group_ids=list(ar_shell.parent_ids), primitives={"text": Texts(texts=[t for t in prompts for _ in range(n_rec)])},
                            sampling_params=req.sampling_params, stage_config={"rollout_id": rid, "mode": "t2t"})
        ar_inner = ar_engine.generate(ar_req).tracks.get(AR_TRACK)
        rec = getattr(ar_inner, "decoded", None)
        if rec is None or len(rec.texts) != len(ar_shell.sample_ids):
            raise RuntimeError(f"UnifiedModelTrainer: the AR engine must return one decoded text per request row ({len(ar_shell.sample_ids)} expected)")
        ar_track = ar_shell.replace(segment=ar_inner.segment, decoded=rec, conditions=dict(ar_inner.conditions))
        img_shell = ar_track.fork_track(parent_name=AR_TRACK, child_name=IMAGE_TRACK, branch=n_img)
        n_ar = len(ar_shell.sample_ids)
        dit_req = RolloutReq(sample_ids=list(img_shell.sample_ids), group_ids=list(img_shell.parent_ids),
                             primitives={"text": Texts(texts=[prompts[i // n_rec] for i in range(n_ar) for _ in range(n_img)]),
                                         "cot_text": Texts(texts=[rec.texts[i] for i in range(n_ar) for _ in range(n_img)])},
                             sampling_params=req.sampling_params, stage_config={"rollout_id": rid, "mode": "t2i"},
                             init_noise_group_ids=[f"r{rid}:{sid}" for sid in img_shell.sample_ids])
        img_inner = dit_engine.generate(dit_req).tracks.get(IMAGE_TRACK)
        if img_inner is None or len(img_inner.sample_ids) != len(img_shell.sample_ids):
            raise RuntimeError(f"UnifiedModelTrainer: the DiT engine must return one image per request row ({len(img_shell.sample_ids)} expected)")
        img_track = img_shell.replace(segment=img_inner.segment, decoded=img_inner.decoded, conditions=dict(img_inner.conditions),
                                      media_preview=getattr(img_inner, "media_preview", None))
        return RolloutResp(tracks={AR_TRACK: ar_track, IMAGE_TRACK: img_track})

    # ---- weight sync choreography -------------------------------------------------------------------------------
    def _engines(self) -> List[Any]:
        return self.ar_rollouts + self.dit_rollouts

    def _extract_then_offload(self) -> None:
        """Trainer resident, engines asleep: gather what the engines need, then give the device memory back."""
        if self._enable_fsdp_offload:
            self.backend.onload()
        if self.weight_sync is not None:
            self.weight_sync.extract()
        if self._enable_fsdp_offload and not self._engine_syncs:
            self.backend.offload()

    def _push(self) -> Dict[str, float]:
        from unirl_b200.distributed.utils import Broadcast
        from unirl_b200.distributed.weight_sync.lora.remote import _Opaque

        t0 = time.perf_counter()
        stats: Dict[str, float] = {}
        if self.weight_sync is not None:
            payload = self.weight_sync.push()[0].value
            for eng in self._engines():
                eng.set_lora_from_tensors(Broadcast(payload["adapter_name"]), Broadcast(_Opaque(payload["tensors"])), peft_config=Broadcast(payload["peft_config"]))
            stats = {"tensors": float(len(payload["tensors"])), "weight_version": float(payload["version"])}
        for ws in self._engine_syncs:  # handlers that move whole weights need trainer and engine resident together
            out = ws.sync()
            stats.update(out[0] if isinstance(out, list) else out)
        if self._engine_syncs and self._enable_fsdp_offload:
            self.backend.offload()
        stats["sync_ms"] = (time.perf_counter() - t0) * 1e3
        return stats

    def _dump(self, rollout_id: int, resp: Any, req: Optional[RolloutReq] = None) -> None:
        """Inspection dump of one rollout: per track one row per sample (id, parent, reward, text), plus the images as a tensor file."""
        if not self.rollout_dump_dir:
            return
        try:
            os.makedirs(self.rollout_dump_dir, exist_ok=True)
            rows = []
            for name, t in resp.tracks.items():
                texts = getattr(t.decoded, "texts", None)
                rw = None if t.rewards is None else hydrate_if_handle(t.rewards)
                for i, sid in enumerate(t.sample_ids):
                    rows.append({"track": name, "sample_id": sid, "parent_id": None if not t.parent_ids else t.parent_ids[i],
                                 "reward": None if rw is None else float(rw[i]), "text": texts[i] if texts is not None else None})
                px = getattr(t.decoded, "pixels", None)
                if px is not None:
                    import torch

                    px = hydrate_if_handle(px)
                    torch.save({"sample_ids": list(t.sample_ids), "pixels": px.detach().cpu()}, os.path.join(self.rollout_dump_dir, f"rollout_{rollout_id:06d}_{name}.pt"))
            if req is not None and "text" in req.primitives:
                rows.insert(0, {"track": "prompts", "texts": list(req.primitives["text"].texts)})
            with open(os.path.join(self.rollout_dump_dir, f"rollout_{rollout_id:06d}.jsonl"), "w") as f:
                for r in rows:
                    f.write(json.dumps(r) + "\n")
        except Exception as e:  # noqa: BLE001 - a dump never breaks training
            logger.warning("rollout dump failed: %s", e)

    # ---- one step -------------------------------------------------------------------------------------------
    def train_step(self, req: RolloutReq, *, training_progress: float = 0.0, sync_weights: bool = False, rollout_id: int = 0) -> Tuple[Any, float]:
        if self.two_engines:
            return self._train_step_two_engines(req, training_progress=training_progress, sync_weights=sync_weights, rollout_id=rollout_id)
        t0 = time.perf_counter()
        self.rollout.wake_up()
        if sync_weights and self.weight_sync is not None:
            self.weight_sync.sync()
        resp = self.rollout.generate(req)
        self.rollout.sleep()
        leaf = IMAGE_TRACK if IMAGE_TRACK in resp.tracks else AR_TRACK
        resp.tracks[leaf] = self.reward.score_and_attach(req=req, track=resp.tracks[leaf])
        rewards = hydrate_if_handle(resp.tracks[leaf].rewards)
        resp.tracks[leaf].rewards = rewards
        if leaf == IMAGE_TRACK and AR_TRACK in resp.tracks:  # the rewrite is judged by the image it led to
            resp.tracks[AR_TRACK].rewards = rewards.clone()
        self._dump(rollout_id, resp)
        tracks = {}
        for name, t in resp.tracks.items():
            t = t.compute_advantages(normalize=self.normalize_adv_by_std, scope=self.adv_normalization_scope)
            t.decoded = None
            tracks[name] = resp.tracks[name] = t
        result = self.stack.train_tracks(tracks.get(AR_TRACK), tracks.get(IMAGE_TRACK), training_progress=float(training_progress))
        self.wandb_logger.log_rollout_step(rollout_id, result, resp.metadata_only(), step_time_s=time.perf_counter() - t0,
                                           device_ms=dict(self.phase_timer.device_ms))
        return result, float(rewards.float().mean())

    def _train_step_two_engines(self, req: RolloutReq, *, training_progress: float, sync_weights: bool, rollout_id: int) -> Tuple[Any, float]:
        from unirl_b200.types.sampling import get_ar_params

        t0 = time.perf_counter()
        self._rollout_id = int(rollout_id)
        sync_stats: Dict[str, float] = {}
        # steady state on entry: engines asleep; with offload enabled the trainer's state is on the host
        if sync_weights and (self.weight_sync is not None or self._engine_syncs):
            self._extract_then_offload()
        for eng in self._engines():
            eng.wake_up()
        if sync_weights and (self.weight_sync is not None or self._engine_syncs):
            sync_stats = self._push()
        resp = self.run_rollout(req)
        for eng in self._engines():
            eng.sleep()
        if self._enable_fsdp_offload:
            self.backend.onload()
        # score the images against their ORIGINAL prompt (one prompt per image, so the request shards together with the track)
        img = resp.tracks[IMAGE_TRACK]
        ar_p, d_p = get_ar_params(req.sampling_params), get_diffusion_params(req.sampling_params)
        fan = (int(ar_p.samples_per_prompt) if ar_p is not None else 1) * int(d_p.samples_per_prompt)
        prompts = req.primitives["text"].texts
        reward_texts = [prompts[i // fan] for i in range(len(img.sample_ids))]
        reward_req = RolloutReq(sample_ids=list(img.sample_ids), group_ids=list(img.parent_ids or img.sample_ids), primitives={"text": Texts(texts=reward_texts)},
                                sampling_params=req.sampling_params, metadata=[])
        scored = self.reward.score_and_attach(req=reward_req, track=img)
        scored.rewards = hydrate_if_handle(scored.rewards)
        resp.tracks[IMAGE_TRACK] = scored
        resp = resp.propagate_rewards(op="mean")  # a rewrite earns the mean reward of the images it led to
        mean_reward = float(resp.tracks[IMAGE_TRACK].rewards.float().mean())
        self._dump(rollout_id, resp, req)
        for name in (AR_TRACK, IMAGE_TRACK):
            resp.tracks[name] = resp.tracks[name].compute_advantages(normalize=self.normalize_adv_by_std, scope=self.adv_normalization_scope)
        self._drop_decoded(req, resp, rollout_id=rollout_id, media_prompts={IMAGE_TRACK: reward_texts})
        result = self.stack.train_tracks(resp.tracks[AR_TRACK], resp.tracks[IMAGE_TRACK], training_progress=float(training_progress))
        self.wandb_logger.log_rollout_step(rollout_id, result, resp.metadata_only(), step_time_s=time.perf_counter() - t0, sync_stats=sync_stats,
                                           device_ms=dict(self.phase_timer.device_ms))
        if self._enable_fsdp_offload:
            self.backend.offload()  # back to the steady state: the next rollout's engines find the memory free
        return result, mean_reward

    def train(self, *, num_rollouts: int, weight_sync_interval: int = 1, save_interval: int = 0, save_dir: Optional[str] = None,
              load_dir: Optional[str] = None, save_mode: str = "full") -> None:
        if self._enable_fsdp_offload and load_dir:
            self.backend.onload()
        start = self.maybe_load_checkpoint(load_dir, num_rollouts=num_rollouts)
        for _ in range(start):
            self.data_source.get_samples(self.batch_size)
        self._init_wandb(num_rollouts=num_rollouts)
        try:
            for rid in range(start, num_rollouts):
                req = self._build_req(self.data_source.get_samples(self.batch_size), rid)
                # engines with weights of their own start from the trainer's: the first step syncs as well
                sync = (self.two_engines and rid == start) or (rid > 0 and rid % max(1, weight_sync_interval) == 0)
                result, mean_reward = self.train_step(req, training_progress=rid / max(1, num_rollouts - 1), sync_weights=sync, rollout_id=rid)
                self.wandb_logger.log_progress(rid, num_rollouts, result, mean_reward, logger=logger)
                if self._enable_fsdp_offload and save_interval > 0:
                    self.backend.onload()
                self.maybe_save_checkpoint(rid, num_rollouts, save_interval=save_interval, save_dir=save_dir, save_mode=save_mode)
                if self._enable_fsdp_offload and save_interval > 0:
                    self.backend.offload()
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
