"""Cross-component recipe validators: checks that span several recipe nodes and are cheap to run before any worker starts.

Each validator raises ``ConfigValidationError`` with the offending keys; ``validate_recipe`` runs all that apply.
Parity: ``unirl/config/validation.py`` (defined there, not wired to a call site; here ``main_entry`` calls
``validate_recipe`` when ``validate: true`` is set or ``UNIRL_B200_VALIDATE=1``).
"""

from __future__ import annotations

from typing import Any, Callable, List


class ConfigValidationError(ValueError):
    pass


def _get(node: Any, dotted: str, default: Any = None) -> Any:
    cur = node
    for part in dotted.split("."):
        if cur is None:
            return default
        cur = cur.get(part) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


def validate_batch_geometry(cfg: Any) -> None:
    """Prompts × samples must split over the data-parallel ranks and the micro-batches."""
    n_dev, bs = int(_get(cfg, "num_devices", 1)), int(_get(cfg, "batch_size", 1))
    spp = int(_get(cfg, "sampling.samples_per_prompt", 0) or 0)
    if not spp:
        spp = int(_get(cfg, "sampling.diffusion.samples_per_prompt", 1)) * int(_get(cfg, "sampling.ar.samples_per_prompt", 1))
    sp = int(_get(cfg, "train_parallel.sp", 1))
    dp = max(1, n_dev // sp)
    if (bs * spp) % dp:
        raise ConfigValidationError(f"batch_size*samples_per_prompt = {bs * spp} does not split over {dp} data-parallel ranks (num_devices={n_dev}, sp={sp})")
    updates = int(_get(cfg, "stack.num_updates_per_batch", 1))
    if ((bs * spp) // dp) % updates:
        raise ConfigValidationError(f"per-rank batch {(bs * spp) // dp} does not split into stack.num_updates_per_batch={updates} mini-batches")


def validate_rollout_parallelism(cfg: Any) -> None:
    tp_cfg, tp_par = int(_get(cfg, "rollout.config.tp_size", 1)), int(_get(cfg, "rollout_parallel.tp", 1))
    if tp_cfg != tp_par:
        raise ConfigValidationError(f"rollout.config.tp_size={tp_cfg} but rollout_parallel.tp={tp_par}")
    if int(_get(cfg, "num_devices", 1)) % max(1, tp_par):
        raise ConfigValidationError(f"rollout tp={tp_par} does not divide num_devices={_get(cfg, 'num_devices', 1)}")


def validate_sampling_consistency(cfg: Any) -> None:
    """Engine-side and request-side generation limits must agree; SDE indices must lie inside the schedule."""
    e, s = _get(cfg, "rollout.config.max_new_tokens"), _get(cfg, "sampling.max_new_tokens")
    if e is not None and s is not None and int(s) > int(e):
        raise ConfigValidationError(f"sampling.max_new_tokens={s} exceeds rollout.config.max_new_tokens={e}")
    steps, idx = _get(cfg, "sampling.num_inference_steps"), _get(cfg, "sampling.sde_indices")
    if steps is not None and idx is not None and any(int(i) < 0 or int(i) >= int(steps) for i in idx):
        raise ConfigValidationError(f"sampling.sde_indices={list(idx)} outside the {steps}-step schedule")
    g_s, g_a = _get(cfg, "sampling.guidance_scale"), _get(cfg, "algorithm.params.guidance_scale")
    if g_s is not None and g_a is not None and float(g_s) != float(g_a):
        raise ConfigValidationError(f"rollout guidance {g_s} != replay guidance {g_a}: replay would score another policy")


def validate_lora_sync(cfg: Any) -> None:
    lora = _get(cfg, "backend.lora_cfg") or _get(cfg, "backend.ema_lora_cfg")
    sync = str(_get(cfg, "sync._target_", ""))
    if lora is None and "Lora" in sync:
        raise ConfigValidationError(f"{sync} needs backend.lora_cfg / backend.ema_lora_cfg")
    if str(_get(cfg, "algorithm._target_", "")).endswith("DiffusionNFT") and _get(cfg, "backend.ema_lora_cfg") is None:
        raise ConfigValidationError("DiffusionNFT needs backend.ema_lora_cfg (trainable + EMA adapter pair)")


def validate_algorithm_horizon(cfg: Any) -> None:
    h, m = _get(cfg, "algorithm.horizon"), _get(cfg, "sampling.max_new_tokens")
    if h is not None and m is not None and int(h) < int(m):
        raise ConfigValidationError(f"algorithm.horizon={h} is shorter than sampling.max_new_tokens={m}")


def validate_train_topology(cfg: Any) -> None:
    """Parallel degrees the trainers do not execute are refused up front instead of being silently ignored: pipeline stages (the
    dispatch layer rejects them for auto-backward anyway).  Sequence parallelism (DiT) and context parallelism (autoregressive replay)
    share the placement dimension ``train_parallel.sp``: the ranks of such a group receive the same samples; the backend option
    (``fsdp_cfg.sp_size`` or ``fsdp_cfg.cp_size``) says which of the two the model runs.  The degree must divide the device count."""
    for key in ("train_parallel.pp", "train_parallel.cp", "backend.topology.pp_size", "backend.topology.cp_size"):
        v = _get(cfg, key)
        if v is not None and int(v) > 1:
            raise ConfigValidationError(f"{key}={v}: this degree is not executed by any trainer (use dp / sp / tp / ep; context parallelism is "
                                        "backend.fsdp_cfg.cp_size with train_parallel.sp)")
    sp = int(_get(cfg, "train_parallel.sp", 1))
    if sp > 1 and int(_get(cfg, "num_devices", 1)) % sp:
        raise ConfigValidationError(f"train_parallel.sp={sp} does not divide num_devices={_get(cfg, 'num_devices', 1)}")
    fs, fc = int(_get(cfg, "backend.fsdp_cfg.sp_size", 1) or 1), int(_get(cfg, "backend.fsdp_cfg.cp_size", 1) or 1)
    if fs > 1 and fc > 1:
        raise ConfigValidationError("backend.fsdp_cfg.sp_size and cp_size are not combined")
    if max(fs, fc) != sp and (max(fs, fc) > 1 or sp > 1):
        raise ConfigValidationError(f"backend.fsdp_cfg.sp_size={fs} / cp_size={fc} but train_parallel.sp={sp}")


VALIDATORS: List[Callable[[Any], None]] = [validate_train_topology, validate_batch_geometry, validate_rollout_parallelism, validate_sampling_consistency, validate_lora_sync,
                                            validate_algorithm_horizon]


def validate_recipe(cfg: Any) -> None:
    problems = []
    for v in VALIDATORS:
        try:
            v(cfg)
        except ConfigValidationError as e:
            problems.append(str(e))
    if problems:
        raise ConfigValidationError("; ".join(problems))


__all__ = ["ConfigValidationError", "validate_recipe", "VALIDATORS", "validate_batch_geometry", "validate_rollout_parallelism", "validate_sampling_consistency",
           "validate_lora_sync", "validate_algorithm_horizon", "validate_train_topology"]
