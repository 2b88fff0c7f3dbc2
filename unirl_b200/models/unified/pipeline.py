"""Bundle and pipeline of the unified (text + image in one transformer) families.

Request modes (``req.stage_config["mode"]``):

``t2t`` / ``i2t``   text out: one ``"ar"`` track (``i2t`` prepends the source image as clean latent context — here: its latents
                    travel as an ``ImageLatentCondition`` and condition the prompt through the codec).
``t2i`` / ``it2i``  image out: one ``"image"`` track; with ``recaption=True`` the model first rewrites the prompt (an ``"ar"``
                    track, trained jointly) and the image is conditioned on ``prompt ⊕ rewrite``.
Parity: ``unirl/models/hunyuan_image3/pipeline.py`` (4 modes, fused multimodal condition), ``unirl/models/bagel/pipeline.py``.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from unirl_b200.models.dit.diffusion import DiTDiffusionParams
from unirl_b200.models.dit.vae import LatentVAE, VAEConfig
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.models.types import Bundle, Pipeline
from unirl_b200.models.unified.modeling import UnifiedConfig, UnifiedTransformer
from unirl_b200.models.unified.stages import UnifiedARStage, UnifiedConditions, UnifiedDiffusionStage
from unirl_b200.sde.runtime import FlowMatchSchedulePolicy, ensure_req_sigmas
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.conditions.base import Modality
from unirl_b200.types.noise_recipe import NoiseRecipe
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack
from unirl_b200.types.sampling import ARSamplingParams, get_ar_params, get_diffusion_params
from unirl_b200.utils.dtypes import parse_torch_dtype

PRESETS = {"tiny-unified": UnifiedConfig.tiny, "tiny-mot": lambda: UnifiedConfig.tiny(name="tiny-mot", num_experts=0, modality_experts=True),
           "hunyuan-image3": UnifiedConfig.hunyuan_image3, "bagel-7b": UnifiedConfig.bagel_7b}


@dataclass
class UnifiedPipelineConfig:
    pretrained_model_ckpt_path: str = "random:tiny-unified"
    model_precision: Any = "bf16"
    device: Any = None
    autocast_precision: str = "bf16"
    trajectory_precision: str = "fp32"
    use_gradient_checkpointing: bool = False
    shift: float = 3.0
    max_prompt_length: int = 512
    negative_prompt: str = ""
    recaption: bool = False
    init_seed: int = 0
    model_overrides: Dict[str, Any] = field(default_factory=dict)
    weight_sync_param_name_prefix: str = "transformer."


class UnifiedBundle(Bundle):
    def __init__(self, transformer: UnifiedTransformer, vae: LatentVAE, tokenizer: Any, config: UnifiedPipelineConfig):
        super().__init__()
        self.transformer, self.vae, self.tokenizer, self.config = transformer, vae, tokenizer, config
        self.modality = Modality.IMAGE
        self.pretrained_path = None

    @property
    def model_config(self) -> UnifiedConfig:
        return self.transformer.cfg

    @classmethod
    def from_config(cls, config: UnifiedPipelineConfig) -> "UnifiedBundle":
        path = config.pretrained_model_ckpt_path
        if not path.startswith("random:"):
            raise NotImplementedError("UnifiedBundle builds random-init presets; checkpoint import for the 80B MoE is per-rank shard loading and is not wired yet")
        mcfg = PRESETS[path.split(":", 1)[1].lower()]()
        for k, v in (config.model_overrides or {}).items():
            setattr(mcfg, k, v)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = UnifiedTransformer(mcfg, dtype=parse_torch_dtype(config.model_precision), device=device,
                                   gradient_checkpointing=config.use_gradient_checkpointing).init_weights(config.init_seed)
        vcfg = VAEConfig.tiny(mcfg.latent_channels) if mcfg.hidden_size <= 256 else VAEConfig(latent_channels=mcfg.latent_channels)
        return cls(model, LatentVAE(vcfg, device=device).init_weights(config.init_seed + 7), load_tokenizer(None, mcfg.vocab_size, True), config)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


class UnifiedPipeline(Pipeline):
    conditions_cls = UnifiedConditions

    def __init__(self, bundle: UnifiedBundle):
        super().__init__()
        self.bundle = bundle
        self.ar = UnifiedARStage(bundle)
        self.diffusion = UnifiedDiffusionStage(bundle, "flow", bundle.config.autocast_precision)
        self.image = self.diffusion  # the image track's stage
        self.shift = float(bundle.config.shift)

    @classmethod
    def from_bundle(cls, bundle: UnifiedBundle, **_kw: Any) -> "UnifiedPipeline":
        return cls(bundle)

    @classmethod
    def from_config(cls, config: UnifiedPipelineConfig) -> "UnifiedPipeline":
        return cls(UnifiedBundle.from_config(config))

    def build_schedule_policy(self) -> FlowMatchSchedulePolicy:
        c = self.bundle.model_config
        return FlowMatchSchedulePolicy(shift=self.shift, vae_scale_factor=self.bundle.vae.cfg.spatial_factor, patch_size=c.patch_size)

    def latent_shape(self, sampling: Any) -> Tuple[int, ...]:
        d = get_diffusion_params(sampling)
        f = self.bundle.vae.cfg.spatial_factor
        return (self.bundle.model_config.latent_channels, int(d.height) // f, int(d.width) // f)

    def _tokens(self, strs: List[str]) -> TextTokenCondition:
        c, tok = self.bundle.model_config, self.bundle.tokenizer
        rows = [[int(x) % c.vocab_size for x in tok.encode(s)][: self.bundle.config.max_prompt_length] or [int(c.pad_token_id)] for s in strs]
        width = max(len(r) for r in rows)
        ids = torch.full((len(rows), width), int(c.pad_token_id), dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : len(r)], mask[i, : len(r)] = torch.tensor(r), 1
        return TextTokenCondition(input_ids=ids, attention_mask=mask)

    def generate(self, req: RolloutReq) -> RolloutResp:
        mode = str((req.stage_config or {}).get("mode", "t2i"))
        if mode not in ("t2t", "i2t", "t2i", "it2i"):
            raise ValueError(f"unknown mode {mode!r}")
        texts = req.primitives.get("text")
        strs = [t.to_str() for t in texts.to_list()]
        tracks: Dict[str, RolloutTrack] = {}
        image_cond = (req.request_conditions or {}).get("image")
        cot = req.primitives.get("cot_text")  # a rewrite produced elsewhere (the AR engine of a two-engine rollout): condition on it, do not regenerate
        wants_text = mode in ("t2t", "i2t") or (bool(self.bundle.config.recaption) and cot is None)
        if cot is not None:
            strs = [f"{s} {c.to_str()}".strip() for s, c in zip(strs, cot.to_list())]
        if wants_text:
            ar = get_ar_params(req.sampling_params) or ARSamplingParams(max_new_tokens=32)
            conds = UnifiedConditions(prompt=self._tokens(strs), image=image_cond)
            seg = self.ar.autoregress(conds, sampling_params=ar)
            cu = seg.cu_seqlens.tolist()
            outs = [self.bundle.tokenizer.decode(seg.tokens[cu[i] : cu[i + 1]].tolist(), skip_special_tokens=True) for i in range(len(cu) - 1)]
            tracks["ar"] = RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids), conditions=conds.to_dict(), segment=seg,
                                        decoded=Texts(texts=outs))
            strs = [f"{s} {o}".strip() for s, o in zip(strs, outs)]
        if mode in ("t2i", "it2i"):
            d = get_diffusion_params(req.sampling_params)
            ensure_req_sigmas(req, self.build_schedule_policy())
            conds = UnifiedConditions(prompt=self._tokens(strs), image=image_cond)
            if float(d.guidance_scale) > 1.0:
                conds.negative_prompt = self._tokens([self.bundle.config.negative_prompt] * len(strs))
            shape = tuple(req.init_noise_latent_shape) if req.init_noise_latent_shape else self.latent_shape(d)
            recipe = NoiseRecipe.from_rollout_req(req).for_batch(req.batch_size, latent_shape=shape)
            if not recipe.noise_group_ids:
                recipe.noise_group_ids = list(req.group_ids if d.init_same_noise else req.sample_ids)
            params = DiTDiffusionParams(guidance_scale=float(d.guidance_scale), eta=float(d.eta), strategy=d.sde_strategy,
                                        trajectory_precision=self.bundle.config.trajectory_precision)
            seg = self.diffusion.diffuse(conds, schedule=req.sigmas, params=params, initial_noise=recipe.resolve(device="cpu"),
                                         sde_indices=d.resolve_sde_indices(int((req.stage_config or {}).get("rollout_id", 0))),
                                         sample_ids=list(req.sample_ids), seed=int(d.seed or 0))
            px = self.bundle.vae.decode(seg.latents[:, -1].float())
            tracks["image"] = RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids), conditions=conds.to_dict(), segment=seg,
                                           decoded=Images(pixels=px.cpu()))
        return RolloutResp(tracks=tracks)


__all__ = ["UnifiedPipelineConfig", "UnifiedBundle", "UnifiedPipeline", "PRESETS"]
