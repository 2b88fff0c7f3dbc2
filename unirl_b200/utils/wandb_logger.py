"""Metrics logging and phase timing.

``UniRLWandBLogger`` keeps the reference's metric namespaces and step axes — ``train/*`` against
``train/step`` (optimizer steps), ``rollout/*`` / ``perf/*`` / ``sync/*`` / ``buffer/*`` against ``rollout/step``,
``eval/*`` — and degrades to stdout + an in-memory history when wandb reporting is off
(``unirl/utils/wandb_logger.py:318-334`` axes, ``log_rollout_step`` flattening).

``PhaseTimer`` / ``install_phase_timing`` wrap the trainer's collaborator calls named in
``STEP_PHASE_SPECS`` (``:43-79``, ``:85-92``, ``:95-142``).  Handle calls are blocking barriers, so host
wall-clock brackets them correctly; in addition, when the controller process owns a CUDA device
(spmd / inline backends) each phase is also bracketed by CUDA events and reported as
``perf/<phase>_device_ms`` — the device-timed figure the benchmarks use.
"""

from __future__ import annotations

import functools
import json
import logging
import os
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from unirl_b200.utils.timing import PhaseTimings

_log = logging.getLogger(__name__)

STEP_PHASE_SPECS: Tuple[Tuple[str, str, str], ...] = (
    ("rollout", "wake_up", "wake"), ("rollout", "generate", "rollout"), ("rollout", "sleep", "sleep"),
    ("weight_sync", "sync", "sync"), ("reward", "score_and_attach", "reward"), ("stack", "train_track", "train"),
    ("backend", "onload", "onload"), ("backend", "offload", "offload"),
)
_STEP_PHASE_SPECS = STEP_PHASE_SPECS


from unirl_b200.utils.profiling import nvtx_range  # noqa: E402


class PhaseTimer:
    def __init__(self) -> None:
        self.timings = PhaseTimings()
        self.device_ms: Dict[str, float] = {}
        self._cuda = torch.cuda.is_available()

    def reset(self) -> None:
        self.timings = PhaseTimings()
        self.device_ms = {}

    def wrap(self, phase: str, fn: Callable[..., Any]) -> Callable[..., Any]:
        @functools.wraps(fn)
        def timed(*a: Any, **k: Any) -> Any:
            ev = None
            if self._cuda:
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            t0 = time.perf_counter()
            try:
                with nvtx_range(f"phase/{phase}"):
                    return fn(*a, **k)
            finally:
                self.timings.add(phase, time.perf_counter() - t0)
                if ev is not None:
                    ev[1].record()
                    ev[1].synchronize()
                    self.device_ms[phase] = self.device_ms.get(phase, 0.0) + ev[0].elapsed_time(ev[1])

        timed._phase_timed = True  # type: ignore[attr-defined]
        return timed


def install_phase_timing(trainer: Any) -> PhaseTimer:
    """Wrap ``trainer.train_step`` and (lazily, at the first step) the collaborator methods of ``STEP_PHASE_SPECS``."""
    timer = PhaseTimer()
    trainer.phase_timer = timer
    inner = trainer.train_step

    def _wrap_collaborators() -> None:
        for attr, method, phase in STEP_PHASE_SPECS:
            obj = getattr(trainer, attr, None)
            fn = getattr(obj, method, None) if obj is not None else None
            if callable(fn) and not getattr(fn, "_phase_timed", False):
                setattr(obj, method, timer.wrap(phase, fn))

    from unirl_b200.utils.profiling import ProfileWindow

    cfg = getattr(trainer, "cfg", None)
    window = ProfileWindow.from_cfg(cfg.get("profile") if hasattr(cfg, "get") else None)
    trainer.profile_window = window
    calls = [0]

    @functools.wraps(inner)
    def train_step(*a: Any, **k: Any) -> Any:
        _wrap_collaborators()
        timer.reset()
        window.step_begin(calls[0])
        t0 = time.perf_counter()
        try:
            with nvtx_range(f"train_step/{calls[0]}"):
                out = inner(*a, **k)
        finally:
            window.step_end(calls[0])
            calls[0] += 1
        timer.timings.step_time_s = time.perf_counter() - t0
        trainer.last_phase_timings = timer.timings
        return out

    trainer.train_step = train_step
    return timer


class UniRLWandBLogger:
    def __init__(self, enabled: bool = False, run: Any = None, log_media: bool = False, media_max_items: int = 8, media_log_interval: int = 1,
                 optimizer_step: int = 0, log_dir: Optional[str] = None) -> None:
        self.enabled, self.run = bool(enabled) and run is not None, run
        self.log_media, self.media_max_items, self.media_log_interval = log_media, int(media_max_items), max(1, int(media_log_interval))
        self.optimizer_step = int(optimizer_step)
        self.history: List[Dict[str, Any]] = []
        self._jsonl = open(os.path.join(log_dir, "metrics.jsonl"), "a") if log_dir and os.path.isdir(log_dir) else None

    @property
    def initialized(self) -> bool:
        return self.enabled

    @property
    def run_id(self) -> Optional[str]:
        return getattr(self.run, "id", None)

    def _emit(self, row: Dict[str, Any]) -> None:
        self.history.append(row)
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({k: v for k, v in row.items() if isinstance(v, (int, float, str))}) + "\n")
            self._jsonl.flush()
        if self.enabled:
            self.run.log(row)

    def should_log_media(self, rollout_id: int) -> bool:
        return self.enabled and self.log_media and (rollout_id + 1) % self.media_log_interval == 0

    def log_generated_media(self, step: int, preview: Any, key: str = "rollout/generated_media") -> None:
        if not self.enabled or preview is None or preview.thumbs is None:
            return
        import wandb

        imgs = [wandb.Image(t.permute(1, 2, 0).numpy(), caption=c) for t, c in zip(preview.thumbs.reshape(-1, *preview.thumbs.shape[-3:]), preview.captions)]
        self.run.log({key: imgs, "rollout/step": step})

    def log_rollout_step(self, rollout_id: int, result: Any, resp: Any, *, step_time_s: float, trunc_len: Optional[int] = None,
                         timings: Optional[PhaseTimings] = None, sync_stats: Optional[Dict[str, float]] = None,
                         device_ms: Optional[Dict[str, float]] = None, roofline: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        step = rollout_id + 1
        row: Dict[str, Any] = {"rollout/step": step, "perf/step_time_s": float(step_time_s)}
        n_samples = n_tokens = 0
        for name, track in getattr(resp, "tracks", {}).items():
            pre = "rollout/" if len(resp.tracks) == 1 else f"rollout/{name}/"
            n_samples = max(n_samples, len(track.sample_ids))
            if isinstance(track.rewards, torch.Tensor) and track.rewards.numel():
                r = track.rewards.float()
                row[pre + "reward_mean"], row[pre + "reward_std"] = float(r.mean()), float(r.std()) if r.numel() > 1 else 0.0
            if isinstance(track.component_rewards, dict):
                for k, v in track.component_rewards.items():
                    if isinstance(v, torch.Tensor) and v.numel():
                        row[pre + f"reward/{k}"] = float(v.float().mean())
            if isinstance(track.advantages, torch.Tensor) and track.advantages.numel():
                a = track.advantages.float()
                row[pre + "advantage_abs_mean"], row[pre + "advantage_max"] = float(a.abs().mean()), float(a.max())
            lens = getattr(track.segment, "lengths", None) if track.segment is not None else None
            if isinstance(lens, torch.Tensor) and lens.numel():
                n_tokens += int(lens.sum())
                row[pre + "response_length_mean"], row[pre + "response_length_max"] = float(lens.float().mean()), float(lens.max())
                if trunc_len:
                    row[pre + "truncation_rate"] = float((lens >= int(trunc_len)).float().mean())
        if timings is not None:
            row.update(timings.as_perf_dict(n_samples or None, n_tokens or None))
        elif step_time_s > 0 and n_samples:
            row["perf/samples_per_s"] = n_samples / step_time_s
            if n_tokens:
                row["perf/tokens_per_s"] = n_tokens / step_time_s
        for k, v in (device_ms or {}).items():
            row[f"perf/{k}_device_ms"] = float(v)
        for k, v in (sync_stats or {}).items():
            row[f"sync/{k}"] = float(v)
        if roofline and device_ms:
            # device-timed phases against the measured peaks: kernel/train_roofline_frac, kernel/decode_roofline_frac (utils/profiling.py)
            from unirl_b200.utils.profiling import roofline_metrics

            lens_all = [getattr(t.segment, "lengths", None) for t in getattr(resp, "tracks", {}).values() if t.segment is not None]
            lens_all = [x for x in lens_all if isinstance(x, torch.Tensor) and x.numel()]
            if lens_all:
                resp_lens = torch.cat([x.float().cpu() for x in lens_all])
                prompt_mean = float(roofline.get("prompt_len_mean", 0.0))
                row.update(roofline_metrics(n_params=int(roofline["n_params"]), train_tokens=int(resp_lens.sum() + prompt_mean * resp_lens.numel()),
                                            train_ms=float(device_ms.get("train", 0.0)), decode_tokens=int(resp_lens.sum()), decode_steps=int(resp_lens.max()),
                                            rollout_ms=float(device_ms.get("rollout", 0.0)), kv_bytes_per_token=int(roofline.get("kv_bytes_per_token", 0)),
                                            mean_context=prompt_mean + float(resp_lens.max()) / 2, batch=int(roofline.get("decode_batch", resp_lens.numel())),
                                            weight_bytes=roofline.get("weight_bytes")))
        self._emit(row)
        per_update = getattr(result, "per_update", ()) or ({**dict(getattr(result, "metrics", {})), "loss": getattr(result, "loss", 0.0),
                                                            "grad_norm": getattr(result, "grad_norm", 0.0)},)
        for upd in per_update:
            self.optimizer_step += 1
            trow = {"train/step": self.optimizer_step, "train/lr": float(getattr(result, "lr", 0.0))}
            for k, v in upd.items():
                if isinstance(v, (list, tuple)) and v and all(isinstance(x, (int, float)) for x in v):
                    v = sum(v) / len(v)
                if isinstance(v, (int, float)) and not isinstance(v, bool):
                    trow[f"train/{k}"] = float(v)
            self._emit(trow)
        return row

    def log_eval(self, step: int, metrics: Dict[str, float]) -> None:
        self._emit({"eval/step": step, **{f"eval/{k}": float(v) for k, v in metrics.items()}})

    def log_progress(self, rollout_id: int, num_rollouts: int, result: Any, mean_reward: float, logger: Optional[logging.Logger] = None) -> None:
        msg = (f"rollout {rollout_id + 1}/{num_rollouts}  loss={getattr(result, 'loss', 0.0):.6f}  grad_norm={getattr(result, 'grad_norm', 0.0):.4f}  "
               f"lr={getattr(result, 'lr', 0.0):.3e}  reward={mean_reward:.4f}")
        (logger or _log).info(msg)
        print(msg, flush=True)

    def finish(self) -> None:
        if self._jsonl is not None:
            self._jsonl.close()
            self._jsonl = None
        if self.enabled:
            self.run.finish()


def init_logger(*, project: Optional[str], run_name: Optional[str] = None, config: Optional[Dict[str, Any]] = None, log_dir: Optional[str] = None,
                rank: int = 0, tags: Optional[List[str]] = None, entity: Optional[str] = None, log_media: bool = False, media_max_items: int = 8,
                media_log_interval: int = 1, enabled: bool = False, run_id: Optional[str] = None, optimizer_step: int = 0) -> UniRLWandBLogger:
    run = None
    if enabled and rank == 0 and project:
        import wandb

        run = wandb.init(project=project, name=run_name, config=config, dir=log_dir, tags=tags, entity=entity, id=run_id,
                         resume="allow" if run_id else None, mode=os.environ.get("WANDB_MODE", "offline"))
        for ns, axis in (("train/*", "train/step"), ("rollout/*", "rollout/step"), ("perf/*", "rollout/step"), ("sync/*", "rollout/step"),
                         ("buffer/*", "rollout/step"), ("eval/*", "eval/step")):
            run.define_metric(axis)
            run.define_metric(ns, step_metric=axis)
    return UniRLWandBLogger(enabled=run is not None, run=run, log_media=log_media, media_max_items=media_max_items,
                            media_log_interval=media_log_interval, optimizer_step=optimizer_step, log_dir=log_dir)


__all__ = ["UniRLWandBLogger", "PhaseTimer", "install_phase_timing", "init_logger", "STEP_PHASE_SPECS"]
