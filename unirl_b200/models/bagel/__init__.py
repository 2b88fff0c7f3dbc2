"""Bagel: unified mixture-of-transformers text-to-image model — every layer holds one parameter set for text /
understanding tokens and one for generated-image tokens (hard routing by modality), image generation by flow matching on
latent patch tokens.  Built on :mod:`unirl_b200.models.unified` with ``modality_experts=True``; the flow forward runs with
gradients enabled for training.

What the family adds to the unified core (``unirl/models/bagel/diffusion.py:66-110`` and the guidance of its flow forward):

* **guidance only inside a window of the schedule**: the text-guidance scale applies while ``cfg_interval[0] < σ <= cfg_interval[1]``,
  outside it the step is a single conditional pass;
* **renormalised guidance**: the guided velocity is scaled back towards the norm of the conditional one —
  ``scale = clamp(|v_cond| / |v_guided|, cfg_renorm_min, 1)`` with the norms taken over everything of a sample (``global``) or per token
  over the channels (``channel`` / ``text_channel``);
* its sampling record carries those knobs next to the common ones, so one ``sampling`` object serves the trainer and the stage.

Parity: ``unirl/models/bagel/{bundle,diffusion,rl_ops}.py``."""
from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch

from unirl_b200.config.require import require
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, as_stage_params
from unirl_b200.models.unified import UnifiedBundle, UnifiedConditions, UnifiedPipeline, UnifiedPipelineConfig
from unirl_b200.models.unified.stages import UnifiedDiffusionStage
from unirl_b200.types.sampling import DiffusionSamplingParams

CFG_RENORM_TYPES = ("global", "channel", "text_channel")


@dataclass
class BagelPipelineConfig(UnifiedPipelineConfig):
    pretrained_model_ckpt_path: str = "random:bagel-7b"


@dataclass
class BagelDiffusionParams(DiffusionSamplingParams):
    """Sampling record of the family: the common fields with Bagel's defaults, plus the guidance knobs of its flow forward."""

    num_inference_steps: int = 14
    guidance_scale: float = 1.0
    height: int = 512
    width: int = 512
    eta: float = 1.0
    cfg_text_scale: float = 1.0
    cfg_img_scale: float = 1.0
    cfg_interval: Tuple[float, float] = (0.0, 1.0)
    cfg_renorm_min: float = 0.0
    cfg_renorm_type: str = "global"
    cfg_type: str = "parallel"

    def __post_init__(self) -> None:
        super().__post_init__()
        require(int(self.num_inference_steps) >= 2, f"BagelDiffusionParams.num_inference_steps must be at least 2, got {self.num_inference_steps}")
        require(self.cfg_renorm_type in CFG_RENORM_TYPES, f"BagelDiffusionParams.cfg_renorm_type must be one of {CFG_RENORM_TYPES}, got {self.cfg_renorm_type!r}")


@dataclass
class BagelStageParams(DiTDiffusionParams):
    cfg_interval: Tuple[float, float] = (0.0, 1.0)
    cfg_renorm_min: float = 0.0
    cfg_renorm_type: str = "global"


class BagelDiffusionStage(UnifiedDiffusionStage):
    def _stage_params(self, params: Any) -> BagelStageParams:
        if isinstance(params, BagelStageParams):
            return params
        base = as_stage_params(params)
        get = (lambda k, d: params.get(k, d)) if isinstance(params, dict) else (lambda k, d: getattr(params, k, d))
        text_scale = float(get("cfg_text_scale", 1.0) or 1.0)
        lo, hi = get("cfg_interval", (0.0, 1.0)) or (0.0, 1.0)
        return BagelStageParams(**{**base.__dict__, "guidance_scale": text_scale if text_scale > 1.0 else base.guidance_scale}, cfg_interval=(float(lo), float(hi)),
                                cfg_renorm_min=float(get("cfg_renorm_min", 0.0) or 0.0), cfg_renorm_type=str(get("cfg_renorm_type", "global") or "global"))

    def _branches(self, x: torch.Tensor, sigma: torch.Tensor, cond: UnifiedConditions, p: DiTDiffusionParams):
        lo, hi = getattr(p, "cfg_interval", (0.0, 1.0))
        s = float(sigma.reshape(-1)[0])
        if not (lo < s <= hi):  # outside the guidance window: one conditional pass
            m = self.bundle.transformer
            t = sigma.to(x.device).float().reshape(-1).expand(x.shape[0]) * 1000.0
            return m.forward_image(cond.prompt.input_ids.to(x.device), cond.prompt.attention_mask.to(x.device), x, t).float(), None
        return super()._branches(x, sigma, cond, p)

    def _guided(self, v_uncond: torch.Tensor, v_cond: torch.Tensor, p: DiTDiffusionParams) -> torch.Tensor:
        vg = v_uncond + p.guidance_scale * (v_cond - v_uncond)
        kind = getattr(p, "cfg_renorm_type", "global")
        dims = tuple(range(1, vg.dim())) if kind == "global" else (1,)  # latents are [B, C, H, W]: channels at dim 1
        nc, ng = torch.linalg.vector_norm(v_cond, dim=dims, keepdim=True), torch.linalg.vector_norm(vg, dim=dims, keepdim=True)
        return vg * (nc / (ng + 1e-8)).clamp(min=float(getattr(p, "cfg_renorm_min", 0.0)), max=1.0)


class BagelBundle(UnifiedBundle):
    pass


class BagelPipeline(UnifiedPipeline):
    def __init__(self, bundle: Any, **options: Any):
        super().__init__(bundle, **options)
        self.diffusion = self.image = BagelDiffusionStage(bundle, self.diffusion.default_strategy, bundle.config.autocast_precision)

    @classmethod
    def from_config(cls, config: BagelPipelineConfig) -> "BagelPipeline":
        return cls(BagelBundle.from_config(config))


BagelConditions = BagelDiffusionConditions = UnifiedConditions

__all__ = ["BagelPipelineConfig", "BagelBundle", "BagelPipeline", "BagelConditions", "BagelDiffusionConditions", "BagelDiffusionParams", "BagelStageParams", "BagelDiffusionStage", "CFG_RENORM_TYPES"]
