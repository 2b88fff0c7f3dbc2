"""``DiTDiffusionStage`` — denoising loop (rollout), per-step replay (training) and single-step velocity prediction.

Rollout ``diffuse``:  x_T from the request's noise recipe → for every step ``i`` of the pinned σ schedule run the
transformer (one batched ``[uncond, cond]`` pass under classifier-free guidance), then either the stochastic
transition of the configured :class:`StepStrategy` (steps in ``sde_indices``; fused kernel emits ``x_{i+1}``, the
transition mean and its Gaussian log-prob in one pass) or the deterministic Euler step.  Only the latents training needs
are kept: ``x_i`` and ``x_{i+1}`` of every SDE step (trajectory trimming), plus the final sample.

Per-sample determinism: the SDE noise of step ``i`` for a sample is drawn on CPU in fp32 from a generator seeded by
``(base seed, sample id, i)``, so any re-batching of the same request reproduces the same trajectory.

Training ``replay``:  for the requested steps recompute velocity at ``x_i`` with gradients and evaluate the transition
density at the stored ``x_{i+1}``; returns ``ReplayResult(log_probs [B, S], prev_sample_means [B, S, …])``.

Parity: ``unirl/models/sd3/diffusion.py:41-133`` (step), ``:287-407`` (diffuse), ``:413-497`` (replay);
``unirl/models/wan21/diffusion.py:340-468``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.types import ReplayResult
from unirl_b200.ops.sde_step import sde_step
from unirl_b200.sde.kernels import StepStrategy, make_strategy
from unirl_b200.sde.noise import step_noise_seed
from unirl_b200.types.conditions import TextEmbedCondition
from unirl_b200.types.segments.latent import LatentSegment
from unirl_b200.utils.dtypes import parse_torch_dtype


@dataclass
class DiTDiffusionParams:
    guidance_scale: float = 4.5
    eta: float = 1.0
    sigma_max: float = 0.99
    strategy: Any = None  # StepStrategy | name | None (family default)
    trajectory_precision: str = "fp32"
    distilled_guidance_scale: Optional[float] = None
    true_cfg: bool = True  # False: guidance is an input embedding of the model, one pass per step


def as_stage_params(params: Any) -> "DiTDiffusionParams":
    """Stage parameters from whatever a recipe handed over: the stage's own dataclass, ``None`` (defaults), or the request-side sampling
    parameters (recipes written for the reference pass ``params: ${sampling}``), whose matching fields are taken over."""
    if isinstance(params, DiTDiffusionParams):
        return params
    if params is None:
        return DiTDiffusionParams()
    get = (lambda k: params.get(k)) if isinstance(params, dict) else (lambda k: getattr(params, k, None))
    kw = {k: get(k) for k in ("guidance_scale", "eta", "sigma_max", "trajectory_precision", "distilled_guidance_scale", "true_cfg") if get(k) is not None}
    strategy = get("strategy") if get("strategy") is not None else get("sde_strategy")
    return DiTDiffusionParams(strategy=strategy, **kw)


_ODE = StepStrategy()  # deterministic Euler transition for the steps outside the SDE set


def _strategy(obj: Any, default: str) -> StepStrategy:
    if isinstance(obj, StepStrategy):
        return obj
    return make_strategy(str(obj or default))


class DiTDiffusionStage:
    def __init__(self, bundle: Any, default_strategy: str = "cps", autocast_precision: str = "bf16"):
        self.bundle = bundle
        self.default_strategy = default_strategy
        self.autocast_dtype = parse_torch_dtype(autocast_precision)

    def trainable_module(self) -> torch.nn.Module:
        return self.bundle.transformer

    @property
    def device(self) -> torch.device:
        return next(self.bundle.transformer.parameters()).device

    # ---- one velocity evaluation ---------------------------------------------------------------------------
    def _velocity(self, x: torch.Tensor, sigma: torch.Tensor, cond: DiTConditions, p: DiTDiffusionParams) -> torch.Tensor:
        """Guided velocity at ``(x, σ)``; ``σ`` is ``[B]`` in ``[0, 1]`` (the transformer sees ``1000·σ``)."""
        vc, vu = self._branches(x, sigma, cond, p)
        return vc if vu is None else self._guided(vu, vc, p)

    def _stage_params(self, params: Any) -> DiTDiffusionParams:
        """The stage's parameter record from what the caller passed (families with knobs of their own override)."""
        return as_stage_params(params)

    @property
    def _plain_guidance(self) -> bool:
        """True when the family uses the textbook combination ``v_u + g·(v_c − v_u)``, which the SDE-step kernel can form itself."""
        return type(self)._guided is DiTDiffusionStage._guided

    def _step_inputs(self, x: torch.Tensor, sigma: torch.Tensor, cond: DiTConditions, p: DiTDiffusionParams):
        """``(noise_pred, keyword arguments)`` for :func:`sde_step`: with plain guidance the two branches go to the kernel separately."""
        vc, vu = self._branches(x, sigma, cond, p)
        if vu is None:
            return vc, {}
        if self._plain_guidance:
            return vc, {"noise_pred_uncond": vu, "guidance_scale": float(p.guidance_scale)}
        return self._guided(vu, vc, p), {}

    def _branches(self, x: torch.Tensor, sigma: torch.Tensor, cond: DiTConditions, p: DiTDiffusionParams) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """One transformer evaluation at ``(x, σ)``: ``(v_cond, v_uncond)`` from one batched pass under classifier-free guidance,
        ``(v, None)`` otherwise."""
        model = self.bundle.transformer
        t = sigma.to(x.device).float().reshape(-1).expand(x.shape[0]) * 1000.0
        txt = cond.text
        inp = self._model_input(x, cond)
        guidance = None
        if model.cfg.guidance_embed:
            g = p.distilled_guidance_scale if p.distilled_guidance_scale is not None else p.guidance_scale
            guidance = torch.full((x.shape[0],), float(g) * 1000.0, device=x.device)
        use_cfg = p.true_cfg and p.guidance_scale > 1.0 and cond.negative_text is not None
        ie = getattr(cond, "image_embed", None)
        ie = None if (ie is None or ie.embeds is None) else ie.embeds.to(x.device)  # image-encoder tokens: the same for both guidance branches
        extra = {} if ie is None else {"image_embeds": ie}
        if not use_cfg:
            return model(inp, t, txt.embeds, txt.pooled, txt.attn_mask, guidance, **extra).float(), None
        neg = cond.negative_text
        width = max(txt.embeds.shape[1], neg.embeds.shape[1])
        pad = lambda e: torch.nn.functional.pad(e, (0, 0, 0, width - e.shape[1]))  # noqa: E731
        padm = lambda m, e: None if m is None else torch.nn.functional.pad(m, (0, width - e.shape[1]))  # noqa: E731
        emb = torch.cat([pad(neg.embeds), pad(txt.embeds)])
        pooled = None if txt.pooled is None else torch.cat([neg.pooled, txt.pooled])
        mask = None if txt.attn_mask is None or neg.attn_mask is None else torch.cat([padm(neg.attn_mask, neg.embeds), padm(txt.attn_mask, txt.embeds)])
        extra = {} if ie is None else {"image_embeds": torch.cat([ie, ie])}
        v = model(torch.cat([inp, inp]), torch.cat([t, t]), emb, pooled, mask, None if guidance is None else torch.cat([guidance, guidance]), **extra).float()
        vu, vc = v.chunk(2)
        return vc, vu

    def _model_input(self, x: torch.Tensor, cond: DiTConditions) -> torch.Tensor:
        """What the transformer sees for the latent ``x`` (families override): image-to-video bundles append the conditioning image's
        latents along the channel axis."""
        if cond.image is not None and cond.image.latents is not None and getattr(self.bundle, "concat_image_latents", False):
            return torch.cat([x, cond.image.latents.to(x)], 1)
        return x

    def _guided(self, v_uncond: torch.Tensor, v_cond: torch.Tensor, p: DiTDiffusionParams) -> torch.Tensor:
        """Classifier-free guidance combination (families override, e.g. norm-corrected CFG)."""
        return v_uncond + p.guidance_scale * (v_cond - v_uncond)

    # ---- rollout --------------------------------------------------------------------------------------------
    @torch.no_grad()
    def diffuse(self, conditions: DiTConditions, *, schedule: torch.Tensor, params: DiTDiffusionParams, initial_noise: torch.Tensor,
                sde_indices: Optional[Sequence[int]] = None, sample_ids: Optional[List[str]] = None, seed: int = 0) -> LatentSegment:
        dev = self.device
        params = self._stage_params(params)
        sig = schedule.to(dev).float()
        steps = sig.numel() - 1
        sde = sorted(int(i) for i in (range(steps) if sde_indices is None else sde_indices)) if params.eta > 0 else []
        strategy = _strategy(params.strategy, self.default_strategy)
        strategy.reset()
        strategy.init_schedule(sig)
        x = initial_noise.to(dev).float()
        b = x.shape[0]
        ids = list(sample_ids) if sample_ids else [str(i) for i in range(b)]
        keep = sorted(set(sde) | {i + 1 for i in sde} | {steps})
        tdt = parse_torch_dtype(params.trajectory_precision)
        stored = {0: x.to(tdt)} if 0 in keep else {}
        logps, means = [], []
        cond = conditions.to_device(dev) if hasattr(conditions, "to_device") else conditions
        for i in range(steps):
            fused = i in sde and tdt == torch.float32
            with torch.autocast(dev.type, dtype=self.autocast_dtype, enabled=self.autocast_dtype != torch.float32 and dev.type == "cuda"):
                v, cfg_kw = self._step_inputs(x, sig[i], cond, params) if fused else (self._velocity(x, sig[i], cond, params), {})
            if i in sde:
                noise = torch.stack([torch.randn(x.shape[1:], dtype=torch.float32, generator=torch.Generator().manual_seed(step_noise_seed(seed, sid, i)))
                                     for sid in ids]).to(dev)
                if fused:  # the guidance combination, the transition and its log-prob in one pass over the latent
                    x, logp, mean = sde_step(strategy, v, x, sig[i], sig[i + 1], eta=params.eta, sigma_max=params.sigma_max, step_index=i, noise=noise, **cfg_kw)
                else:  # the stored sample is rounded to the trajectory dtype BEFORE its log-prob is taken, so replay sees the same value
                    x, logp, mean = strategy.denoise(v, x.to(tdt), sig[i], sig[i + 1], eta=params.eta, sigma_max=params.sigma_max, step_index=i, noise=noise)
                logps.append(logp.float())
                means.append(mean.to(tdt))
            else:
                x, _, _ = _ODE.denoise(v, x, sig[i], sig[i + 1], step_index=i)
            x = x.float()
            if i + 1 in keep:
                stored[i + 1] = x.to(tdt)
        order = sorted(stored)
        return LatentSegment(modality=self.bundle.modality, latents=torch.stack([stored[k] for k in order], 1), sigmas=sig.cpu(),
                             indices=torch.tensor(order, dtype=torch.long), sde_logp=torch.stack(logps, 1) if logps else None,
                             sde_means=torch.stack(means, 1) if means else None, sde_indices=torch.tensor(sde, dtype=torch.long) if sde else None)

    # ---- training -------------------------------------------------------------------------------------------
    def replay(self, conditions: DiTConditions, *, segment: LatentSegment, params: DiTDiffusionParams, step_indices: Optional[List[int]] = None) -> ReplayResult:
        dev = self.device
        params = self._stage_params(params)
        sig = segment.sigmas.to(dev).float()
        steps = [int(i) for i in (step_indices if step_indices is not None else segment.sde_indices.tolist())]
        strategy = _strategy(params.strategy, self.default_strategy)
        strategy.reset()
        strategy.init_schedule(sig)
        cond = conditions.to_device(dev) if hasattr(conditions, "to_device") else conditions
        logps, means = [], []
        for i in steps:
            x, nxt = segment.latents_at(i).to(dev).float(), segment.latents_at(i + 1).to(dev).float()
            with torch.autocast(dev.type, dtype=self.autocast_dtype, enabled=self.autocast_dtype != torch.float32 and dev.type == "cuda"):
                v, cfg_kw = self._step_inputs(x, sig[i], cond, params)
            _, logp, mean = sde_step(strategy, v, x, sig[i], sig[i + 1], eta=params.eta, prev_sample=nxt, sigma_max=params.sigma_max, step_index=i, **cfg_kw)
            logps.append(logp.float())
            means.append(mean.float())
        return ReplayResult(log_probs=torch.stack(logps, 1), prev_sample_means=torch.stack(means, 1))

    def predict_noise_at_step(self, conditions: DiTConditions, *, sample: torch.Tensor, sigma: torch.Tensor, params: DiTDiffusionParams) -> torch.Tensor:
        dev = self.device
        cond = conditions.to_device(dev) if hasattr(conditions, "to_device") else conditions
        with torch.autocast(dev.type, dtype=self.autocast_dtype, enabled=self.autocast_dtype != torch.float32 and dev.type == "cuda"):
            return self._velocity(sample.to(dev).float(), sigma, cond, self._stage_params(params))


__all__ = ["DiTDiffusionStage", "DiTDiffusionParams", "as_stage_params"]
