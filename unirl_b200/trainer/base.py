"""``BaseTrainer`` — device pool, logger, phase timing, checkpoint save / resume.

Parity: ``unirl/trainer/base.py:52-331`` — pool bring-up from ``cfg.num_devices``; always-present logger
(null object when reporting is off); ``_drop_decoded`` (media preview then free decoded payloads before the
train dispatch); ``maybe_save_checkpoint`` → ``<save_dir>/checkpoint-<step>/checkpoint.pt`` + ``trainer_state.json``;
``maybe_load_checkpoint`` → restored step, wandb run re-attach, optimizer-step axis.
"""

from __future__ import annotations

import json
import logging
import os
from typing import Any, Dict, List, Optional

from unirl_b200.distributed.group.device_pool import DevicePool
from unirl_b200.utils.wandb_logger import UniRLWandBLogger, init_logger, install_phase_timing

logger = logging.getLogger(__name__)


def init_transfer_queue(cfg: Any) -> None:
    """The queue transport needs no controller/storage actors on one box (see ``tensor/backend/transfer_queue.py``)."""
    return None


class BaseTrainer:
    def __init__(self, *, cfg: Any, logging_cfg: Any = None, pool: Optional[DevicePool] = None) -> None:
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        self.cfg = cfg
        self.num_devices = int(get("num_devices", 1) or 1)
        self._owns_pool = pool is None
        backend = get("pool_backend")
        in_torchrun = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1
        spmd = backend == "spmd" or (backend is None and in_torchrun)
        self.pool = pool or DevicePool(gpus_per_node=None if spmd else self.num_devices,
                                       backend=backend, tensor_transport=get("transport_kind", "colocate_store"),
                                       device=get("pool_device"), call_timeout_s=float(get("call_timeout_s", 3600.0)))
        self.logging_cfg = logging_cfg
        self.wandb_logger = UniRLWandBLogger(enabled=False)
        self._resume_state: Dict[str, Any] = {}
        self.last_phase_timings = None
        if self.pool.tensor_transport in ("transfer_queue", "tq"):
            inner = self.train_step

            def _with_reclaim(*a: Any, **k: Any) -> Any:
                out = inner(*a, **k)
                self.pool.reset_transfer_queue_buffers()
                return out

            self.train_step = _with_reclaim
        install_phase_timing(self)

    def train_step(self, *a: Any, **k: Any) -> Any:  # pragma: no cover - subclasses override
        raise NotImplementedError

    # ---- logging ----------------------------------------------------------------------------------------
    def _init_wandb(self, *, num_rollouts: Optional[int] = None, extra: Optional[Dict[str, Any]] = None) -> None:
        c = self.logging_cfg or {}
        get = c.get if hasattr(c, "get") else (lambda k, d=None: d)
        report = bool(get("report_to_wandb", False)) and bool(get("project_name"))
        tags = get("tags")
        if isinstance(tags, str):
            tags = [t.strip() for t in tags.split(",") if t.strip()]
        elif tags:
            tags = [str(t).strip() for t in tags if str(t).strip()]
        sp = getattr(self, "sampling_params", None)
        config = {"num_devices": self.num_devices, "batch_size": getattr(self, "batch_size", None), "num_rollouts": num_rollouts,
                  "samples_per_prompt": getattr(sp, "samples_per_prompt", None), **(extra or {})}
        log_dir = get("logging_dir")
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)
        self.wandb_logger = init_logger(project=str(get("project_name")) if get("project_name") else None, run_name=get("run_name"), config=config,
                                        log_dir=log_dir, rank=self.pool.my_rank, tags=tags or None,
                                        entity=get("entity") or os.environ.get("WANDB_ENTITY") or None, log_media=bool(get("log_media", False)),
                                        media_max_items=int(get("media_max_items", 8)), media_log_interval=int(get("media_log_interval", 1)),
                                        enabled=report, run_id=self._resume_state.get("wandb_run_id"),
                                        optimizer_step=int(self._resume_state.get("optimizer_step") or 0))

    def _finish_wandb(self) -> None:
        if self.wandb_logger is not None:
            self.wandb_logger.finish()

    def _drop_decoded(self, req: Any, resp: Any, *, rollout_id: int, media_prompts: Optional[Dict[str, List[str]]] = None) -> None:
        wb = self.wandb_logger
        if wb is not None and wb.should_log_media(rollout_id):
            from unirl_b200.types.media_preview import build_media_preview_for_track

            multi = len(resp.tracks) > 1
            for name, track in resp.tracks.items():
                preview = track.media_preview
                if preview is None and track.decoded is not None:
                    preview = build_media_preview_for_track(track, max_items=wb.media_max_items, captions=(media_prompts or {}).get(name))
                if preview is not None:
                    wb.log_generated_media(rollout_id + 1, preview, key=f"rollout/{name}/generated_media" if multi else "rollout/generated_media")
        for track in resp.tracks.values():
            track.decoded = None
            track.media_preview = None

    # ---- checkpoints --------------------------------------------------------------------------------------
    def maybe_save_checkpoint(self, rollout_id: int, num_rollouts: int, *, save_interval: int, save_dir: Optional[str], save_mode: str = "full") -> Optional[str]:
        if save_interval <= 0:
            return None
        step = rollout_id + 1
        if step % save_interval != 0 and step < num_rollouts:
            return None
        base = os.path.abspath(save_dir) if save_dir else os.path.join(os.getcwd(), "checkpoints")
        path = os.path.join(base, f"checkpoint-{step}")
        logger.info("saving checkpoint at rollout %d/%d -> %s", step, num_rollouts, path)
        self.backend.save(path, step=step, mode=save_mode)
        if self.pool.my_rank == 0:
            os.makedirs(path, exist_ok=True)
            with open(os.path.join(path, "trainer_state.json"), "w") as f:
                json.dump({"wandb_run_id": self.wandb_logger.run_id, "optimizer_step": self.wandb_logger.optimizer_step, "step": step}, f)
        return path

    def maybe_load_checkpoint(self, load_dir: Optional[str], *, num_rollouts: Optional[int] = None) -> int:
        if not load_dir:
            return 0
        load_dir = os.path.abspath(load_dir)
        steps = self.backend.load(load_dir)
        step = int(steps[0] if isinstance(steps, list) else steps or 0)
        state_path = os.path.join(load_dir, "trainer_state.json")
        if os.path.exists(state_path):
            with open(state_path) as f:
                self._resume_state = json.load(f)
        if num_rollouts is not None and step >= num_rollouts:
            logger.warning("checkpoint step %d already reaches the rollout budget %d", step, num_rollouts)
        logger.info("resumed from %s at rollout step %d", load_dir, step)
        return step

    def shutdown(self) -> None:
        if self._owns_pool:
            self.pool.shutdown()


__all__ = ["BaseTrainer", "init_transfer_queue"]
