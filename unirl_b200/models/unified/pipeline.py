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
    __extra_fields_ok__ = True  # recipes may carry fields of other loaders (config.instantiate.call_target keeps them as attributes)
    pretrained_model_ckpt_path: str = "random:tiny-unified"
    model_precision: Any = "bf16"
    device: Any = None
    autocast_precision: str = "bf16"
    trajectory_precision: str = "fp32"
    logprob_precision: str = "fp32"
    use_gradient_checkpointing: bool = False
    shift: float = 3.0
    guidance_scale: float = 1.0  # default guidance of the image stage when a request does not set one
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

    @staticmethod
    def _model_config(config: UnifiedPipelineConfig) -> UnifiedConfig:
        """``random:<preset>`` or a native checkpoint directory (``config.json`` with ``{"preset": ..., "model": {overrides}}`` next to
        ``model-*.safetensors`` shards and ``model.safetensors.index.json``)."""
        path = config.pretrained_model_ckpt_path
        if path.startswith("random:"):
            mcfg = PRESETS[path.split(":", 1)[1].lower()]()
        else:
            import json
            import os

            with open(os.path.join(path, "config.json")) as f:
                d = json.load(f)
            mcfg = PRESETS[d["preset"]]()
            for k, v in (d.get("model") or {}).items():
                setattr(mcfg, k, v)
        for k, v in (config.model_overrides or {}).items():
            setattr(mcfg, k, v)
        return mcfg

    @classmethod
    def from_meta_config(cls, config: UnifiedPipelineConfig) -> "UnifiedBundle":
        """The bundle with every parameter on the ``meta`` device: shapes and module tree only, no memory.  The 80B mixture-of-experts
        model is built this way on every rank; :meth:`materialize` then allocates and fills what the rank keeps.
        Parity: ``unirl/models/hunyuan_image3/bundle.py:427`` (``from_meta_config``)."""
        mcfg = cls._model_config(config)
        model = UnifiedTransformer(mcfg, dtype=parse_torch_dtype(config.model_precision), device="meta", gradient_checkpointing=config.use_gradient_checkpointing)
        vcfg = VAEConfig.tiny(mcfg.latent_channels) if mcfg.hidden_size <= 256 else VAEConfig(latent_channels=mcfg.latent_channels)
        b = cls(model, LatentVAE(vcfg, device="meta"), load_tokenizer(None, mcfg.vocab_size, True), config)
        b.pretrained_path = None if config.pretrained_model_ckpt_path.startswith("random:") else config.pretrained_model_ckpt_path
        return b

    @torch.no_grad()
    def materialize(self, device: Any, with_aux: bool = True, ep: Any = None) -> "UnifiedBundle":
        """Allocate the parameters on ``device`` and fill them, rank by rank.

        With an expert-parallel context every mixture layer first drops the experts other ranks own (still on ``meta``: nothing was
        allocated for them), so a rank allocates ``1 / P`` of the routed experts plus the shared parameters.  Values come from the
        checkpoint directory -- each rank opens the shards and reads only the tensors it kept, under their GLOBAL names
        (``...experts.<global id>...``) -- or, for ``random:`` presets, from a generator seeded by the tensor's global name, so every
        rank holds the same value for the same tensor whatever the sharding.  ``with_aux=False`` leaves the codec on ``meta`` (ranks
        that never decode).  Parity: ``unirl/models/hunyuan_image3/bundle.py:528`` (``materialize``)."""
        from unirl_b200.models.unified.modeling import MoEFFN

        model = self.transformer
        if ep is not None and getattr(ep, "size", 1) > 1:
            for m in model.modules():
                if isinstance(m, MoEFFN) and m.ep is None:
                    m.shard_experts(ep)
        if any(p.is_meta for p in model.parameters()):
            model.to_empty(device=device)
            global_names = _global_param_names(model)
            if self.pretrained_path is None:
                _init_by_name(model, global_names, int(self.config.init_seed))
            else:
                _load_by_name(model, global_names, self.pretrained_path)
        else:
            model.to(device)
        if with_aux:
            if any(p.is_meta for p in self.vae.parameters()):
                self.vae.to_empty(device=device)
                for n, p in self.vae.named_parameters():  # norm scales and biases: identity / zero; the kernels come from init_weights
                    if p.dim() < 2:
                        p.fill_(1.0 if n.endswith("weight") else 0.0)
                self.vae.init_weights(int(self.config.init_seed) + 7)
            else:
                self.vae.to(device)
        return self

    @classmethod
    def from_config(cls, config: UnifiedPipelineConfig) -> "UnifiedBundle":
        path = config.pretrained_model_ckpt_path
        if not path.startswith("random:"):  # a checkpoint: build on meta, then read the shards straight onto the device
            device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
            return cls.from_meta_config(config).materialize(device)
        mcfg = cls._model_config(config)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = UnifiedTransformer(mcfg, dtype=parse_torch_dtype(config.model_precision), device=device,
                                   gradient_checkpointing=config.use_gradient_checkpointing).init_weights(config.init_seed)
        vcfg = VAEConfig.tiny(mcfg.latent_channels) if mcfg.hidden_size <= 256 else VAEConfig(latent_channels=mcfg.latent_channels)
        return cls(model, LatentVAE(vcfg, device=device).init_weights(config.init_seed + 7), load_tokenizer(None, mcfg.vocab_size, True), config)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


def _global_param_names(model: torch.nn.Module) -> Dict[str, str]:
    """Local parameter name → name in the unsharded model: ``...experts.<slot>...`` becomes ``...experts.<global expert id>...``."""
    from unirl_b200.models.unified.modeling import MoEFFN

    remap: Dict[str, List[int]] = {n: list(m.expert_ids) for n, m in model.named_modules() if isinstance(m, MoEFFN)}
    out: Dict[str, str] = {}
    for name, _ in model.named_parameters():
        g = name
        for mod, ids in remap.items():
            pre = f"{mod}.experts."
            if name.startswith(pre):
                slot, rest = name[len(pre):].split(".", 1)
                g = f"{pre}{ids[int(slot)]}.{rest}"
                break
        out[name] = g
    return out


def _init_by_name(model: torch.nn.Module, global_names: Dict[str, str], seed: int, std: float = 0.02) -> None:
    """Deterministic init keyed on the tensor's global name (not on its position in the module tree, which sharding changes)."""
    import hashlib

    for name, p in model.named_parameters():
        if p.dim() == 1:
            p.fill_(1.0)
            continue
        g = global_names[name]
        h = int.from_bytes(hashlib.blake2b(f"{seed}:{g}".encode(), digest_size=8).digest(), "little") & ((1 << 62) - 1)
        gen = torch.Generator(device="cpu").manual_seed(h)
        vals = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std * (0.25 if g == "patch_out" else 1.0), generator=gen)
        p.copy_(vals.to(p.device))


def _load_by_name(model: torch.nn.Module, global_names: Dict[str, str], path: str) -> None:
    """Read exactly the tensors this rank kept from a sharded safetensors checkpoint (index file: tensor name → shard file)."""
    import json
    import os

    from safetensors import safe_open

    index_file = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index_file):
        with open(index_file) as f:
            where = json.load(f)["weight_map"]
    else:
        where = {}
        for fn in sorted(os.listdir(path)):
            if fn.endswith(".safetensors"):
                with safe_open(os.path.join(path, fn), "pt") as sf:
                    where.update({k: fn for k in sf.keys()})
    by_file: Dict[str, List[Tuple[str, torch.nn.Parameter]]] = {}
    missing = []
    for name, p in model.named_parameters():
        g = global_names[name]
        if g not in where:
            missing.append(g)
            continue
        by_file.setdefault(where[g], []).append((g, p))
    if missing:
        raise KeyError(f"checkpoint {path} lacks {len(missing)} tensors this rank needs, e.g. {missing[:4]}")
    for fn, items in by_file.items():
        with safe_open(os.path.join(path, fn), "pt") as sf:
            for g, p in items:
                t = sf.get_tensor(g)
                if tuple(t.shape) != tuple(p.shape):
                    raise ValueError(f"{g}: checkpoint shape {tuple(t.shape)} vs module {tuple(p.shape)}")
                p.copy_(t.to(p.device, p.dtype))


def save_native_checkpoint(model: torch.nn.Module, path: str, preset: str, overrides: Optional[Dict[str, Any]] = None, shard_bytes: int = 1 << 30) -> None:
    """Write an (unsharded-expert) model as ``config.json`` + ``model-0000k.safetensors`` shards + ``model.safetensors.index.json``."""
    import json
    import os

    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    names = _global_param_names(model)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, p in model.named_parameters():
        nbytes = p.numel() * p.element_size()
        if shards[-1] and size + nbytes > shard_bytes:
            shards.append({})
            size = 0
        shards[-1][names[name]] = p.detach().cpu().contiguous()
        size += nbytes
    weight_map = {}
    for i, sd in enumerate(shards):
        fn = f"model-{i + 1:05d}.safetensors"
        save_file(sd, os.path.join(path, fn))
        weight_map.update({k: fn for k in sd})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": weight_map}, f)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"preset": preset, "model": dict(overrides or {})}, f)


class UnifiedPipeline(Pipeline):
    conditions_cls = UnifiedConditions

    def __init__(self, bundle: UnifiedBundle, *, shift: Optional[float] = None, autocast_precision: Optional[str] = None, **_options: Any):
        super().__init__()
        self.bundle = bundle
        if shift is not None:
            bundle.config.shift = float(shift)
        if autocast_precision is not None:
            bundle.config.autocast_precision = autocast_precision
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


__all__ = ["UnifiedPipelineConfig", "UnifiedBundle", "UnifiedPipeline", "PRESETS", "save_native_checkpoint"]
