"""``DiTPipeline`` — ``RolloutReq`` (prompts) → one ``"diffusion"`` track (conditions, trajectory segment, decoded media).

Order of work: text towers (deduplicated prompts, plus the negative prompt under CFG) → σ schedule pinned on the request
→ x_T from the request's noise recipe (group-seeded CPU fp32 draws, so every engine and the trainer agree byte for byte)
→ :meth:`DiTDiffusionStage.diffuse` → codec decode.  Parity: ``unirl/models/sd3/pipeline.py:97-203``,
``unirl/models/wan21/pipeline.py``.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage
from unirl_b200.models.dit.text_embed import TextEmbedStage
from unirl_b200.models.types import Pipeline
from unirl_b200.sde.runtime import FlowMatchSchedulePolicy, ensure_req_sigmas
from unirl_b200.types.noise_recipe import NoiseRecipe
from unirl_b200.types.primitives import Images, Texts, Videos
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack
from unirl_b200.types.sampling import DiffusionSamplingParams, get_diffusion_params


class DiTPipeline(Pipeline):
    conditions_cls = DiTConditions

    def __init__(self, bundle: DiTBundle, *, shift: Optional[float] = None, autocast_precision: Optional[str] = None, trajectory_precision: Optional[str] = None,
                 logprob_precision: Optional[str] = None, strategy: Any = None, **_ignored: Any):
        """The keyword options are the ones recipes written for the reference pass to a pipeline built directly from its class
        (``pipeline: {_target_: …Pipeline, shift, autocast_precision, trajectory_precision, logprob_precision, strategy}``): they override
        the bundle's configuration; ``strategy`` (a step-strategy object or its name) becomes the family's default SDE strategy."""
        super().__init__()
        self.bundle = bundle
        cfg, spec = bundle.config, bundle.spec
        for name, value in (("shift", shift), ("autocast_precision", autocast_precision), ("trajectory_precision", trajectory_precision),
                            ("logprob_precision", logprob_precision)):
            if value is not None and hasattr(cfg, name):
                setattr(cfg, name, value)
        if strategy is not None:
            from unirl_b200.sde.kernels import STRATEGIES, StepStrategy

            spec.default_strategy = next((k for k, c in STRATEGIES.items() if type(strategy) is c), spec.default_strategy) if isinstance(strategy, StepStrategy) else str(strategy)
        self.text_embed = TextEmbedStage(bundle.text_encoders, bundle.tokenizers, spec.text_combine, spec.transformer.text_dim, cfg.max_sequence_length)
        self.diffusion = DiTDiffusionStage(bundle, spec.default_strategy, cfg.autocast_precision)
        self.shift = float(cfg.shift if cfg.shift is not None else spec.shift)

    @classmethod
    def from_bundle(cls, bundle: DiTBundle, **_kw: Any) -> "DiTPipeline":
        return cls(bundle)

    @classmethod
    def from_config(cls, config: DiTPipelineConfig) -> "DiTPipeline":
        return cls(DiTBundle.from_config(config))

    def build_schedule_policy(self) -> FlowMatchSchedulePolicy:
        return self.bundle.schedule_policy()

    # ---- geometry --------------------------------------------------------------------------------------------
    @classmethod
    def latent_shape_for(cls, spec: Any, d: DiffusionSamplingParams) -> Tuple[int, ...]:
        t = spec.transformer
        h, w = int(d.height) // t.vae_scale_factor, int(d.width) // t.vae_scale_factor
        c = t.out_channels or t.in_channels  # the latent has the transformer's OUTPUT width; extra input channels carry conditioning
        if spec.packed_latents:  # 2x2 spatial patches are folded into channels before the transformer
            h, w = h // 2, w // 2
        if t.is_video:
            return (c, (int(d.num_frames) - 1) // t.vae_temporal_factor + 1, h, w)
        return (c, h, w)

    def latent_shape(self, sampling: Any) -> Tuple[int, ...]:
        return self.latent_shape_for(self.bundle.spec, get_diffusion_params(sampling))

    def _unpack(self, x: torch.Tensor) -> torch.Tensor:
        """Packed latents ``[B, 4c, (F,) h, w]`` → codec latents ``[B, c, (F,) 2h, 2w]``."""
        if not self.bundle.spec.packed_latents:
            return x
        if x.dim() == 4:
            b, c4, h, w = x.shape
            return x.view(b, c4 // 4, 2, 2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(b, c4 // 4, 2 * h, 2 * w)
        b, c4, f, h, w = x.shape
        return x.view(b, c4 // 4, 2, 2, f, h, w).permute(0, 1, 4, 5, 2, 6, 3).reshape(b, c4 // 4, f, 2 * h, 2 * w)

    # ---- generate --------------------------------------------------------------------------------------------
    def _conditions(self, req: RolloutReq, d: DiffusionSamplingParams) -> DiTConditions:
        pre = req.request_conditions or {}
        if "text" in pre:
            return DiTConditions.from_dict(pre)
        texts = req.primitives.get("text")
        if not isinstance(texts, Texts):
            raise TypeError(f"DiTPipeline.generate: req.primitives['text'] must be Texts, got {type(texts).__name__}")
        cond = DiTConditions(text=self.text_embed.embed(texts), image=pre.get("image"))
        if float(d.guidance_scale) > 1.0 and not self.bundle.model_config.guidance_embed:
            n = len(texts)
            cond.negative_text = self.text_embed.embed([self.bundle.config.negative_prompt] * n)
        return cond

    def generate(self, req: RolloutReq) -> RolloutResp:
        d = get_diffusion_params(req.sampling_params)
        ensure_req_sigmas(req, self.build_schedule_policy())
        cond = self._conditions(req, d)
        n = req.batch_size
        shape = tuple(req.init_noise_latent_shape) if req.init_noise_latent_shape else self.latent_shape(d)
        recipe = NoiseRecipe.from_rollout_req(req).for_batch(n, latent_shape=shape)
        if not recipe.noise_group_ids:
            recipe.noise_group_ids = list(req.group_ids if d.init_same_noise else req.sample_ids)
        x_t = recipe.resolve(device="cpu")
        rollout_id = int((req.stage_config or {}).get("rollout_id", 0))
        params = DiTDiffusionParams(guidance_scale=float(d.guidance_scale), eta=float(d.eta), strategy=d.sde_strategy,
                                    trajectory_precision=self.bundle.config.trajectory_precision, distilled_guidance_scale=d.distilled_guidance_scale,
                                    true_cfg=not self.bundle.model_config.guidance_embed)
        seg = self.diffusion.diffuse(cond, schedule=req.sigmas, params=params, initial_noise=x_t, sde_indices=d.resolve_sde_indices(rollout_id),
                                     sample_ids=list(req.sample_ids), seed=int(d.seed or 0))
        decoded = None
        if self.bundle.config.decode_images:
            px = self.bundle.vae.decode(self._unpack(seg.latents[:, -1].float()))
            decoded = Videos.pack(frames=[v.cpu() for v in px]) if px.dim() == 5 else Images(pixels=px.cpu())
        return RolloutResp(tracks={"diffusion": RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids), conditions=cond.to_dict(),
                                                             segment=seg, decoded=decoded)})


__all__ = ["DiTPipeline"]
