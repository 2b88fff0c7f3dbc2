"""``DiffusionTrainer`` — FlowGRPO / Flow-DPPO / DiffusionNFT (and the DanceGRPO / MixGRPO recipes) for flow-matching DiTs.

Same loop as the AR trainer; what differs is the request.  The controller is authoritative for everything that must
agree between rollout and replay and therefore authors it once per rollout:

* the σ schedule (model family's schedule policy, from the light ``FamilySpec`` — no weights needed on the controller),
* the initial-noise recipe (group ids + base seed + latent shape; ``init_same_noise`` shares x_T inside a prompt group),
* the SDE step set (explicit list > window scheduler keyed by the rollout id > every step).

Parity: ``unirl/trainer/diffusion.py`` (request construction, forward-process requests for DiffusionNFT, step loop).
"""

from __future__ import annotations

import dataclasses
import logging
from typing import Any, Optional

from unirl_b200.trainer.ar import ARTrainer
from unirl_b200.types.prompts import RolloutInputs
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.sampling import get_diffusion_params

logger = logging.getLogger(__name__)


def _cfg_get(node: Any, dotted: str, default: Any = None) -> Any:
    cur = node
    for part in dotted.split("."):
        if cur is None:
            return default
        cur = cur.get(part) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


class DiffusionTrainer(ARTrainer):
    track_name = "diffusion"

    def __init__(self, *, cfg: Any, bundle_cfg: Any, **kw: Any) -> None:
        super().__init__(cfg=cfg, bundle_cfg=bundle_cfg, **kw)
        from unirl_b200.config.aliases import translate
        from unirl_b200.models.dit.config import resolve_family
        from unirl_b200.models.dit.pipeline import DiTPipeline

        path = str(_cfg_get(bundle_cfg, "config.pretrained_model_ckpt_path", "random:tiny-sd3"))
        shift = _cfg_get(bundle_cfg, "config.shift")
        # A recipe may name the SDE step strategy on the TRAINER's pipeline (``pipeline.strategy``).  A rollout engine with a pipeline of its
        # own would otherwise sample with its family's default while the trainer replays with the named one, and the two sets of log-probs
        # would describe different transitions: the strategy therefore travels on every request.
        self._strategy_name = self._strategy_of(kw.get("pipeline_cfg"))
        target = translate(str(_cfg_get(bundle_cfg, "_target_", "")))
        if any(f".models.{fam}." in target for fam in ("bagel", "hunyuan_image3", "unified")):
            # a unified text-and-image model trained on its image track only: latent geometry and schedule come from its own configuration
            self._init_unified_geometry(bundle_cfg, shift)
            return
        self._spec = resolve_family(path, dict(_cfg_get(bundle_cfg, "config.model_overrides", {}) or {}))
        self._shape_of = lambda d: DiTPipeline.latent_shape_for(self._spec, d)
        self._policy = self._make_policy(target, shift)

    @staticmethod
    def _strategy_of(pipeline_cfg: Any) -> Optional[str]:
        node = _cfg_get(pipeline_cfg, "strategy") if pipeline_cfg is not None else None
        if node is None:
            return None
        if isinstance(node, str):
            return node
        from unirl_b200.config.instantiate import get_method
        from unirl_b200.sde.kernels import STRATEGIES

        target = _cfg_get(node, "_target_")
        cls = get_method(str(target)) if target else None
        return next((name for name, c in STRATEGIES.items() if c is cls), None)

    def _init_unified_geometry(self, bundle_cfg: Any, shift: Optional[float]) -> None:
        from unirl_b200.config.instantiate import instantiate
        from unirl_b200.models.dit.vae import VAEConfig
        from unirl_b200.models.unified.pipeline import UnifiedBundle
        from unirl_b200.sde.runtime import FlowMatchSchedulePolicy

        conf = instantiate(_cfg_get(bundle_cfg, "config"))
        mcfg = UnifiedBundle._model_config(conf)
        factor = (VAEConfig.tiny(mcfg.latent_channels) if mcfg.hidden_size <= 256 else VAEConfig(latent_channels=mcfg.latent_channels)).spatial_factor
        self._spec = None
        self._shape_of = lambda d: (int(mcfg.latent_channels), int(d.height) // factor, int(d.width) // factor)
        self._policy = FlowMatchSchedulePolicy(shift=float(shift if shift is not None else getattr(conf, "shift", 3.0)), vae_scale_factor=factor, patch_size=mcfg.patch_size)

    def _make_policy(self, bundle_target: str, shift: Optional[float]) -> Any:
        from unirl_b200.sde.runtime import FlowMatchSchedulePolicy

        t = self._spec.transformer
        patch = t.patch_size[-1] * (2 if self._spec.packed_latents else 1)
        kw = dict(shift=float(shift if shift is not None else self._spec.shift), vae_scale_factor=t.vae_scale_factor, patch_size=patch)
        if "flux2_klein" in bundle_target:
            from unirl_b200.models.flux2_klein.schedule import KleinSchedulePolicy

            return KleinSchedulePolicy(**kw)
        return FlowMatchSchedulePolicy(use_dynamic_shifting=self._spec.use_dynamic_shifting, **kw)

    def _build_req(self, inputs: RolloutInputs, rollout_id: int, sampling_params: Any = None) -> RolloutReq:
        sp = sampling_params or self.sampling_params
        d = get_diffusion_params(sp)
        inputs = inputs.expand(sp.samples_per_prompt)
        sde = d.resolve_sde_indices(rollout_id)
        sp = dataclasses.replace(sp, sde_indices=list(sde)) if dataclasses.is_dataclass(sp) and hasattr(sp, "sde_indices") else sp
        if getattr(self, "_strategy_name", None) and dataclasses.is_dataclass(sp) and hasattr(sp, "sde_strategy") and sp.sde_strategy is None:
            sp = dataclasses.replace(sp, sde_strategy=self._strategy_name)
        d = get_diffusion_params(sp)
        sigmas = self._policy.compute_sigma(num_inference_steps=int(d.num_inference_steps), height=int(d.height), width=int(d.width))
        gids = list(inputs.group_ids if d.init_same_noise else inputs.sample_ids)
        return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=dict(inputs.primitives), request_conditions={},
                          sampling_params=sp, sigmas=sigmas, stage_config={"rollout_id": int(rollout_id)},
                          metadata=list(inputs.metadata) if inputs.metadata else [], init_noise_group_ids=gids,
                          init_noise_latent_shape=list(self._shape_of(d)))


__all__ = ["DiffusionTrainer"]
