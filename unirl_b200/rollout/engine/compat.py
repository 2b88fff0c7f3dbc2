"""Engine names of recipes written for the reference, on this package's native engines.

The reference drives external serving stacks: an SGLang language-model server (``SGLangLLMRolloutEngine``), an SGLang diffusion server
(``SGLangRolloutEngine``) and vLLM-Omni (``VLLMOmniRolloutEngine``), each configured by a dataclass of its own.  Here the same work is done in
process by :class:`NativeARRolloutEngine` and :class:`NativeDiffusionRolloutEngine`.  The classes below keep the reference's class and
field names, so a recipe's ``rollout:`` block is read as it stands: fields that carry over are translated, fields that only concern the
external servers (host / port / scheduler endpoints, server warm-up, backend selection) are accepted and have no effect.
``config/instantiate.py`` maps the reference's module paths onto this module.

Parity: ``unirl/rollout/engine/sglang_llm/config.py:23-80``, ``unirl/rollout/engine/sglang/config.py:57-112``,
``unirl/rollout/engine/vllm_omni/config.py:34-71``, ``unirl/rollout/engine/composed/config.py:24-43``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from unirl_b200.rollout.engine.composed.engine import ComposedRolloutEngine
from unirl_b200.rollout.engine.native_ar.config import NativeAREngineConfig
from unirl_b200.rollout.engine.native_ar.engine import NativeARRolloutEngine
from unirl_b200.rollout.engine.native_diffusion.engine import NativeDiffusionEngineConfig, NativeDiffusionRolloutEngine

#: model family of a diffusion recipe → (pipeline class, pipeline configuration class, random-init preset for runs without a checkpoint)
FAMILIES: Dict[str, Tuple[str, str, str]] = {
    "sd3": ("unirl_b200.models.sd3.pipeline.SD3Pipeline", "unirl_b200.models.sd3.config.SD3PipelineConfig", "random:sd35-medium"),
    "wan21": ("unirl_b200.models.wan21.Wan21Pipeline", "unirl_b200.models.wan21.Wan21PipelineConfig", "random:wan21-14b"),
    "wan22": ("unirl_b200.models.wan22.Wan22Pipeline", "unirl_b200.models.wan22.Wan22PipelineConfig", "random:wan21-14b"),
    "qwen_image": ("unirl_b200.models.qwen_image.QwenImagePipeline", "unirl_b200.models.qwen_image.QwenImagePipelineConfig", "random:qwen-image"),
    "flux2_klein": ("unirl_b200.models.flux2_klein.Flux2KleinPipeline", "unirl_b200.models.flux2_klein.Flux2KleinPipelineConfig", "random:flux2-klein"),
    "z_image": ("unirl_b200.models.z_image.ZImagePipeline", "unirl_b200.models.z_image.ZImagePipelineConfig", "random:z-image"),
    "hunyuan_video": ("unirl_b200.models.hunyuan_video.HunyuanVideoPipeline", "unirl_b200.models.hunyuan_video.HunyuanVideoPipelineConfig", "random:hunyuan-video"),
    "hunyuan_video15": ("unirl_b200.models.hunyuan_video15.HunyuanVideo15Pipeline", "unirl_b200.models.hunyuan_video15.HunyuanVideo15PipelineConfig",
                        "random:hunyuan-video15"),
    "hunyuan_image3": ("unirl_b200.models.hunyuan_image3.HunyuanImage3Pipeline", "unirl_b200.models.hunyuan_image3.HunyuanImage3PipelineConfig", "random:hunyuan-image3"),
    "bagel": ("unirl_b200.models.bagel.BagelPipeline", "unirl_b200.models.bagel.BagelPipelineConfig", "random:bagel-7b"),
}

# configuration class of a model family (as recipes pass it to an engine through ``model_config: ${bundle.config}``) → family
_FAMILY_OF_CONFIG = {"SD3PipelineConfig": "sd3", "Wan21PipelineConfig": "wan21", "Wan22PipelineConfig": "wan22", "QwenImagePipelineConfig": "qwen_image",
                     "Flux2KleinPipelineConfig": "flux2_klein", "ZImagePipelineConfig": "z_image", "HunyuanVideoPipelineConfig": "hunyuan_video",
                     "HunyuanVideo15PipelineConfig": "hunyuan_video15", "HunyuanImage3PipelineConfig": "hunyuan_image3", "BagelPipelineConfig": "bagel"}


# ------------------------------------------------------------------------------------------------ language-model engine
@dataclass
class SGLangLLMEngineConfig:
    pretrained_model_ckpt_path: str = ""
    tp_size: Optional[int] = None
    host: Optional[str] = None
    port: Optional[int] = None
    concurrency: int = 8
    samples_pre_expanded: bool = False
    image_token: Optional[str] = None
    max_new_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 1024
    system_instruction: Optional[str] = None
    chat_template_kwargs: Optional[Dict[str, Any]] = field(default_factory=dict)
    engine_kwargs: Optional[Dict[str, Any]] = field(default_factory=dict)
    model_precision: str = "bf16"

    def to_native(self) -> NativeAREngineConfig:
        kw = dict(self.engine_kwargs or {})
        return NativeAREngineConfig(pretrained_model_ckpt_path=self.pretrained_model_ckpt_path or "random:tiny", tp_size=int(self.tp_size or 1),
                                    max_new_tokens=int(self.max_new_tokens), temperature=float(self.temperature), top_p=float(self.top_p), top_k=int(self.top_k),
                                    samples_pre_expanded=bool(self.samples_pre_expanded), concurrency=int(self.concurrency), model_precision=self.model_precision,
                                    max_running_requests=int(kw.get("max_running_requests", kw.get("cuda_graph_max_bs", 256)) or 256),
                                    chat_template_kwargs=dict(self.chat_template_kwargs or {}), engine_kwargs=kw)

    def make_engine(self, **deps: Any) -> "SGLangLLMRolloutEngine":
        return SGLangLLMRolloutEngine(config=self, **deps)


class SGLangLLMRolloutEngine(NativeARRolloutEngine):
    def __init__(self, *, config: Any = None, bundle: Any = None, **overrides: Any) -> None:
        if isinstance(config, dict) and not isinstance(config, NativeAREngineConfig):
            config = SGLangLLMEngineConfig(**config)
        if isinstance(config, SGLangLLMEngineConfig):
            config = config.to_native()
        super().__init__(config=config, bundle=bundle, **overrides)


# ------------------------------------------------------------------------------------------------ diffusion engines
def _diffusion_config(model_path: Optional[str], family: str, *, forward_batch_size: Optional[int], tp_size: Optional[int], init_same_noise: bool = False,
                      use_cuda_graph: bool = True, share_trainer_weights: bool = False, pipeline_overrides: Optional[Dict[str, Any]] = None) -> NativeDiffusionEngineConfig:
    if family not in FAMILIES:
        raise ValueError(f"unknown diffusion model family {family!r}; known: {sorted(FAMILIES)}")
    pipe, pcfg, preset = FAMILIES[family]
    return NativeDiffusionEngineConfig(pipeline_cls=pipe, pipeline_config_cls=pcfg, pretrained_model_ckpt_path=model_path or preset, forward_batch_size=forward_batch_size,
                                       tp_size=int(tp_size or 1), use_cuda_graph=use_cuda_graph, share_trainer_weights=share_trainer_weights,
                                       pipeline_overrides=dict(pipeline_overrides or {}))


@dataclass
class SGLangEngineConfig:
    sampling: Any = None
    model_family: str = "sd3"
    populate_conditions: bool = True
    init_same_noise: bool = False
    num_gpus: int = 1
    tp_size: Optional[int] = None
    sp_degree: Optional[int] = None
    local_mode: bool = True
    disable_autocast: bool = False
    forward_batch_size: Optional[int] = None
    target_modules: Optional[Tuple[str, ...]] = None
    lora_merge_mode: Optional[str] = None
    host: Optional[str] = None
    port: Optional[int] = None
    scheduler_port: Optional[int] = None
    engine_kwargs: Optional[Dict[str, Any]] = field(default_factory=dict)
    pretrained_model_ckpt_path: Optional[str] = None
    share_trainer_weights: Optional[bool] = None  # None: share the trainer's replica when the engine sits on the trainer's devices and is not tensor-parallel

    def to_native(self) -> NativeDiffusionEngineConfig:
        kw = dict(self.engine_kwargs or {})
        path = self.pretrained_model_ckpt_path or kw.get("model_path")
        return _diffusion_config(path, self.model_family, forward_batch_size=self.forward_batch_size, tp_size=self.tp_size, init_same_noise=self.init_same_noise,
                                 use_cuda_graph=not bool(kw.get("disable_cuda_graph", False)), share_trainer_weights=bool(self.share_trainer_weights))

    def make_engine(self, **deps: Any) -> "SGLangRolloutEngine":
        return SGLangRolloutEngine(config=self, **deps)


@dataclass
class VLLMOmniEngineConfig:
    model_path: str = ""
    modality: str = "t2i"
    model_family: str = "sd3"
    default_height: int = 1024
    default_width: int = 1024
    default_num_inference_steps: int = 25
    default_guidance_scale: float = 5.0
    default_eta: float = 1.0
    default_ar_max_tokens: int = 2048
    default_ar_temperature: float = 0.6
    default_ar_top_p: float = 0.95
    default_ar_top_k: int = 1024
    enable_sleep_mode: bool = True
    omni_extra: Dict[str, Any] = field(default_factory=dict)
    forward_batch_size: Optional[int] = None
    tensor_parallel_size: Optional[int] = None

    def to_native(self, family: Optional[str] = None) -> NativeDiffusionEngineConfig:
        # "ar_recaption" / "dit_recaption": the two engines of a unified model, one serving its text stage and one its image stage
        overrides = {"recaption": True} if "recaption" in str(self.modality) else {}
        return _diffusion_config(self.model_path or None, family or self.model_family, forward_batch_size=self.forward_batch_size,
                                 tp_size=self.tensor_parallel_size or self.omni_extra.get("tensor_parallel_size"), pipeline_overrides=overrides)

    def make_engine(self, **deps: Any) -> "VLLMOmniRolloutEngine":
        return VLLMOmniRolloutEngine(config=self, **deps)


class _DiffusionCompat(NativeDiffusionRolloutEngine):
    _config_cls: Any = SGLangEngineConfig

    def __init__(self, *, config: Any = None, pipeline: Any = None, model_config: Any = None, strategy: Any = None, **_deps: Any) -> None:
        """``model_config``: the trainer bundle's configuration record (recipes pass ``${bundle.config}``): the engine's own copy of the
        model is built from the same checkpoint path and precisions.  ``strategy`` rides on the requests here and is not needed."""
        if isinstance(config, dict):
            config = self._config_cls(**config)
        if hasattr(config, "to_native"):
            family = _FAMILY_OF_CONFIG.get(type(model_config).__name__) if model_config is not None else None
            native = config.to_native(family) if family and isinstance(config, VLLMOmniEngineConfig) else config.to_native()
            get = (lambda k: model_config.get(k)) if isinstance(model_config, dict) else (lambda k: getattr(model_config, k, None))
            if model_config is not None:
                explicit = getattr(config, "pretrained_model_ckpt_path", None) or getattr(config, "model_path", None) or (getattr(config, "engine_kwargs", None) or {}).get("model_path")
                if not explicit and get("pretrained_model_ckpt_path"):
                    native.pretrained_model_ckpt_path = str(get("pretrained_model_ckpt_path"))
                for name in ("model_precision", "autocast_precision", "device"):
                    if get(name) is not None:
                        setattr(native, name, get(name))
            if getattr(config, "share_trainer_weights", None) is None and pipeline is not None and int(native.tp_size) == 1:
                native.share_trainer_weights = True  # same devices as the trainer: one replica serves both, weight sync becomes a no-op
            config = native
        super().__init__(config=config, pipeline=pipeline)


class SGLangRolloutEngine(_DiffusionCompat):
    _config_cls = SGLangEngineConfig


class VLLMOmniRolloutEngine(_DiffusionCompat):
    _config_cls = VLLMOmniEngineConfig


# ------------------------------------------------------------------------------------------------ composed engine
@dataclass
class ComposedRolloutEngineConfig:
    ar: Any = None
    diffusion: Any = None
    sleep_diffusion_on_start: bool = True
    pe_instruction: Optional[str] = None
    pe_marker: Optional[str] = None
    pe_max_chars: Optional[int] = None

    def make_engine(self, **deps: Any) -> ComposedRolloutEngine:
        return ComposedRolloutEngine(config=self, **deps)


__all__ = ["FAMILIES", "SGLangLLMEngineConfig", "SGLangLLMRolloutEngine", "SGLangEngineConfig", "SGLangRolloutEngine", "VLLMOmniEngineConfig", "VLLMOmniRolloutEngine",
           "ComposedRolloutEngineConfig"]
