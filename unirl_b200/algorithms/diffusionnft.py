"""DiffusionNFT — forward-process negative-aware fine-tuning with a trainable and an EMA ("old") adapter.

For K timesteps t (the rollout's σ schedule without the terminal 0, sliced by
``training_timestep_fraction``; or uniform random): ``x_t = (1−t)x0 + t·ε``; ``v_new`` from the trainable
adapter, ``v_old`` from the EMA adapter (no grad); implicit positive / negative policies
``v⁺ = βv_new + (1−β)v_old``, ``v⁻ = (1+β)v_old − βv_new``; reconstructed ``x̂0± = x_t − t·v±``; adaptive-weighted
MSE to the clean latent; ``r = clamp(A, ±c)/c/2 + ½``; ``loss = (r·L⁺ + (1−r)·L⁻)/β · c``; one backward per
timestep scaled ``loss_scale/K``.  Parity: ``unirl/algorithms/diffusionnft.py:92-200``, ``:206-296``,
``:302-392``, ``:394-449``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple, Type

import torch

from unirl_b200.algorithms.base import AlgorithmStepResult, BaseAlgorithmConfig, StageAlgorithm, typed_conditions
from unirl_b200.utils.scheduler_utils import normalize_timestep_fraction


@dataclass
class DiffusionNFTConfig(BaseAlgorithmConfig):
    beta: float = 1.0
    adv_clip_max: float = 5.0
    adv_mode: str = "raw"
    use_adaptive_weight: bool = True
    train_timestep_mode: str = "all"
    shuffle_train_timesteps: bool = True
    apply_time_shift_in_loss: bool = False
    training_timestep_fraction: float = 0.99
    kl_coef: float = 0.0


class DiffusionNFT(StageAlgorithm):
    requires_ema_rollout = True
    supports_multi_update = False

    def __init__(self, *, params: Any, stage: Any = None, pipeline: Any = None, stage_attr: str = "diffusion",
                 nft_lora_policy: Any = None, backend: Any = None, beta: float = 1.0, adv_clip_max: float = 5.0,
                 adv_mode: str = "raw", use_adaptive_weight: bool = True, train_timestep_mode: str = "all",
                 shuffle_train_timesteps: bool = True, apply_time_shift_in_loss: bool = False,
                 training_timestep_fraction: float = 0.99, kl_coef: float = 0.0, conditions_cls: Optional[Type[Any]] = None) -> None:
        super().__init__()
        if stage is None and pipeline is not None:
            stage = getattr(pipeline, stage_attr)
        if stage is None:
            raise ValueError("DiffusionNFT: pass `stage` or `pipeline`")
        if nft_lora_policy is None and backend is not None:
            nft_lora_policy = getattr(backend, "ema", None)
        if adv_mode != "raw":
            raise ValueError(f"DiffusionNFT: adv_mode={adv_mode!r} unsupported (only 'raw')")
        if train_timestep_mode not in ("all", "random"):
            raise ValueError(f"DiffusionNFT: train_timestep_mode={train_timestep_mode!r} unsupported")
        if apply_time_shift_in_loss:
            raise ValueError("DiffusionNFT: apply_time_shift_in_loss is not implemented")
        if not 0.0 < float(training_timestep_fraction) <= 1.0:
            raise ValueError("DiffusionNFT: training_timestep_fraction must lie in (0, 1]")
        if float(kl_coef) > 0:
            raise ValueError("DiffusionNFT: kl_coef > 0 is not supported")
        if not float(beta) > 0 or not float(adv_clip_max) > 0:
            raise ValueError("DiffusionNFT: beta and adv_clip_max must be > 0")
        if not callable(getattr(nft_lora_policy, "use_shadow", None)):
            raise TypeError(f"DiffusionNFT: nft_lora_policy={type(nft_lora_policy).__name__} lacks use_shadow()")
        self.stage, self.params, self.nft_lora_policy, self.conditions_cls = stage, params, nft_lora_policy, conditions_cls
        self.config = DiffusionNFTConfig(float(beta), float(adv_clip_max), str(adv_mode), bool(use_adaptive_weight),
                                         str(train_timestep_mode), bool(shuffle_train_timesteps), False,
                                         float(training_timestep_fraction), float(kl_coef))

    # ---- pieces -------------------------------------------------------------------------------------
    def _resolve_timesteps(self, segment: Any, batch: int, device: Any, dtype: torch.dtype) -> torch.Tensor:
        c = self.config
        if c.train_timestep_mode == "random":
            ts = torch.rand(batch, device=device, dtype=dtype) * c.training_timestep_fraction
        else:
            if segment.sigmas is None:
                raise ValueError("DiffusionNFT(train_timestep_mode='all') needs segment.sigmas")
            ts = segment.sigmas.detach().to(device=device, dtype=dtype).flatten()
            if ts.numel() > 1 and abs(float(ts[-1])) < 1e-8:
                ts = ts[:-1]
            if ts.numel() and c.training_timestep_fraction != 1.0:
                lo, hi = normalize_timestep_fraction(c.training_timestep_fraction)
                n = ts.numel()
                ts = ts[int(n * lo) : min(int(n * hi), n)]
            if not ts.numel():
                ts = torch.rand(1, device=device, dtype=dtype) * c.training_timestep_fraction
        if c.shuffle_train_timesteps:
            ts = ts[torch.randperm(ts.numel(), device=device)]
        return ts

    def _loss_at_t(self, conditions: Any, x0: torch.Tensor, t: torch.Tensor, r: torch.Tensor, adv: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, float]]:
        c, b = self.config, x0.shape[0]
        t_b = t.detach().to(device=x0.device, dtype=torch.float32).expand(b)
        t_e = t_b.view(b, *([1] * (x0.dim() - 1)))
        x_t = (1.0 - t_e) * x0 + t_e * torch.randn_like(x0)
        v_new = self.stage.predict_noise_at_step(conditions, sample=x_t, sigma=t_b, params=self.params)
        with torch.no_grad(), self.nft_lora_policy.use_shadow():
            v_old = self.stage.predict_noise_at_step(conditions, sample=x_t, sigma=t_b, params=self.params).detach()
        v_pos = c.beta * v_new + (1.0 - c.beta) * v_old
        v_neg = (1.0 + c.beta) * v_old - c.beta * v_new
        target = x0.to(v_new.dtype)
        dims = tuple(range(1, x0.dim()))
        err_pos, err_neg = (x_t - t_e * v_pos) - target, (x_t - t_e * v_neg) - target
        if c.use_adaptive_weight:
            with torch.no_grad():
                w_pos = err_pos.detach().double().abs().mean(dims, keepdim=True).clamp(min=1e-5).to(v_new.dtype)
                w_neg = err_neg.detach().double().abs().mean(dims, keepdim=True).clamp(min=1e-5).to(v_new.dtype)
            l_pos, l_neg = (err_pos**2 / w_pos).mean(dims), (err_neg**2 / w_neg).mean(dims)
        else:
            l_pos, l_neg = (err_pos**2).mean(dims), (err_neg**2).mean(dims)
        policy = (r * l_pos / c.beta + (1.0 - r) * l_neg / c.beta).mean()
        stats = {"policy_loss": float(policy.detach()), "pos_loss_mean": float(l_pos.mean().detach()),
                 "neg_loss_mean": float(l_neg.mean().detach()), "r_mean": float(r.mean()), "advantage_mean": float(adv.mean()),
                 "advantage_std": float(adv.std()) if b > 1 else 0.0,
                 "prediction_deviation": float(((v_new - v_old) ** 2).mean().detach()), "x0_norm": float((x0**2).mean()),
                 "t_value": float(t)}
        return policy * c.adv_clip_max, stats

    def compute_loss_and_backward(self, *, conditions: Mapping[str, Any], segment: Any, advantages: torch.Tensor,
                                  training_progress: float, loss_scale: float) -> AlgorithmStepResult:
        if segment.latents is None or not segment.latents.shape[0]:
            return AlgorithmStepResult.skipped()
        conds = typed_conditions(conditions, self.conditions_cls)
        x0 = segment.latents[:, -1].float()
        b = x0.shape[0]
        adv = advantages.detach().to(device=x0.device, dtype=torch.float32).reshape(b)
        cmax = self.config.adv_clip_max
        r = (adv.clamp(-cmax, cmax) / cmax / 2.0 + 0.5).clamp(0.0, 1.0)
        ts = self._resolve_timesteps(segment, b, x0.device, torch.float32)
        k = int(ts.numel())
        total, collected = 0.0, []
        for t in ts:
            loss, stats = self._loss_at_t(conds, x0, t, r, adv)
            (loss * (loss_scale / k)).backward()
            total += float(loss.detach())
            collected.append(stats)
        metrics = {key: sum(s[key] for s in collected) / k for key in collected[0]}
        metrics["num_train_timesteps"] = k
        return AlgorithmStepResult(total / k, metrics, k, True)


__all__ = ["DiffusionNFT", "DiffusionNFTConfig"]
