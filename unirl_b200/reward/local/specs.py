"""The reference's recipe convention for reward backends — ``backend: {_target_: …Scorer, base_device, config: {_target_: …Spec, …}}`` —
on this package's scorers.

Every published scorer of the reference has a ``<Name>Spec`` dataclass (pure data: batch size, device, model and processor ids, checkpoint
paths) and a ``<Name>RewardScorer(config=<Spec>, base_device=…)`` class.  The classes below keep those names and fields and build the scorer
of ``scorers.py`` that plays the part; model ids name local checkpoint directories here (no hub access is assumed), and a spec whose model
cannot be found falls back to the small random-init towers so a recipe still runs end to end.  ``config/instantiate.py`` maps the
reference's module paths (``unirl.reward.local.pickscore`` …) onto this module.

Parity: ``unirl/reward/local/{clip,pickscore,hpsv2,hpsv3,image_reward,aesthetic,ocr,geneval2,video,video_pickscore}.py`` (spec fields),
``unirl/reward/base.py:64-73`` (``BaseRewardComponentSpec``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from unirl_b200.reward.local.scorers import AestheticScorer, ClipStyleScorer, GenEvalScorer, OCRScorer, VideoScorer


class BaseRewardComponentSpec:
    """Marker base of the reward backend specs (each spec is a dataclass of its own fields)."""


def _device(spec_device: str, base_device: Optional[str]) -> Optional[str]:
    d = (spec_device or "auto").lower()
    if d != "auto":
        return spec_device
    return None if base_device in (None, "auto") else base_device


def _local_or_none(model_id: Optional[str]) -> Optional[str]:
    """A model id is usable when it names a local checkpoint directory; hub names are not resolved here."""
    return model_id if model_id and os.path.isdir(model_id) else None


@dataclass
class ClipSpec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    model_id: str = "openai/clip-vit-large-patch14"


@dataclass
class PickScoreSpec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    processor_id: str = "laion/CLIP-ViT-H-14-laion2B-s32B-b79K"
    model_id: str = "yuvalkirstain/PickScore_v1"


@dataclass
class HPSv2Spec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    open_clip_path: str = "./hps_ckpt/open_clip_pytorch_model.bin"
    checkpoint_path: str = "./hps_ckpt/HPS_v2.1_compressed.pt"
    model_id: Optional[str] = None  # a transformers-layout export of the HPS towers, when one is at hand


@dataclass
class HPSv3Spec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    model_id: Optional[str] = None


@dataclass
class ImageRewardSpec(BaseRewardComponentSpec):
    device: str = "auto"
    model_version: str = "ImageReward-v1.0"
    batch_size: int = 8


@dataclass
class AestheticSpec(BaseRewardComponentSpec):
    device: str = "auto"


@dataclass
class OCRSpec(BaseRewardComponentSpec):
    lang: str = "en"
    device: str = "auto"


@dataclass
class GenEval2Spec(BaseRewardComponentSpec):
    batch_size: int = 1
    device: str = "auto"
    model_name: str = "Qwen/Qwen3-VL-8B-Instruct"
    data_path: str = ""
    aggregation: str = "gm"


@dataclass
class VideoSpec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    inner_model_name: str = "pickscore"
    temporal_weight: float = 0.3
    alignment_weight: float = 0.7
    sample_frames: int = 8


@dataclass
class VideoPickScoreSpec(BaseRewardComponentSpec):
    batch_size: int = 8
    device: str = "auto"
    processor_id: str = "laion/CLIP-ViT-H-14-laion2B-s32B-b79K"
    model_id: str = "yuvalkirstain/PickScore_v1"
    sample_frames: int = 8


class _ClipFamily(ClipStyleScorer):
    variant_name = "clip"
    spec_cls: Any = ClipSpec

    def __init__(self, *, config: Any = None, base_device: Optional[str] = None, **kw: Any):
        c = config if config is not None else self.spec_cls()
        self.config = c
        super().__init__(self.variant_name, device=_device(getattr(c, "device", "auto"), base_device), model_id=_local_or_none(getattr(c, "model_id", None)),
                         processor_id=_local_or_none(getattr(c, "processor_id", None)), batch_size=int(getattr(c, "batch_size", 8)), **kw)


class ClipRewardScorer(_ClipFamily):
    canonical_model_name = "clip"


class PickScoreRewardScorer(_ClipFamily):
    canonical_model_name = variant_name = "pickscore"
    spec_cls = PickScoreSpec


class HPSv2RewardScorer(_ClipFamily):
    canonical_model_name = variant_name = "hpsv2"
    spec_cls = HPSv2Spec


class HPSv3RewardScorer(_ClipFamily):
    canonical_model_name = variant_name = "hpsv3"
    spec_cls = HPSv3Spec


class ImageRewardScorer(_ClipFamily):
    canonical_model_name = variant_name = "image_reward"
    spec_cls = ImageRewardSpec


class AestheticRewardScorer(AestheticScorer):
    canonical_model_name = "aesthetic"

    def __init__(self, *, config: Optional[AestheticSpec] = None, base_device: Optional[str] = None, **kw: Any):
        self.config = config or AestheticSpec()
        super().__init__(device=_device(self.config.device, base_device), **kw)


class OCRRewardScorer(OCRScorer):
    canonical_model_name = "ocr"

    def __init__(self, *, config: Optional[OCRSpec] = None, base_device: Optional[str] = None, **kw: Any):
        self.config = config or OCRSpec()
        super().__init__(**kw)


class GenEval2RewardScorer(GenEvalScorer):
    canonical_model_name = "geneval2"

    def __init__(self, *, config: Optional[GenEval2Spec] = None, base_device: Optional[str] = None, **_kw: Any):
        self.config = config or GenEval2Spec()


class VideoRewardScorer(VideoScorer):
    canonical_model_name = "video"

    def __init__(self, *, config: Optional[VideoSpec] = None, base_device: Optional[str] = None, **kw: Any):
        c = self.config = config or VideoSpec()
        super().__init__(variant=c.inner_model_name if c.inner_model_name in ClipStyleScorer.VARIANTS else "pickscore", temporal_weight=float(c.temporal_weight),
                         device=_device(c.device, base_device), batch_size=int(c.batch_size), **kw)


class VideoPickScoreScorer(VideoScorer):
    canonical_model_name = "videopickscore"

    def __init__(self, *, config: Optional[VideoPickScoreSpec] = None, base_device: Optional[str] = None, **kw: Any):
        c = self.config = config or VideoPickScoreSpec()
        super().__init__(variant="pickscore", device=_device(c.device, base_device), model_id=_local_or_none(c.model_id), processor_id=_local_or_none(c.processor_id),
                         batch_size=int(c.batch_size), **kw)


#: scorer name → (scorer class, spec class), the registry the reference keeps in ``reward/local/registry.py``
REGISTRY: Dict[str, Tuple[type, type]] = {
    "clip": (ClipRewardScorer, ClipSpec), "pickscore": (PickScoreRewardScorer, PickScoreSpec), "hpsv2": (HPSv2RewardScorer, HPSv2Spec),
    "hpsv3": (HPSv3RewardScorer, HPSv3Spec), "image_reward": (ImageRewardScorer, ImageRewardSpec), "aesthetic": (AestheticRewardScorer, AestheticSpec),
    "ocr": (OCRRewardScorer, OCRSpec), "geneval2": (GenEval2RewardScorer, GenEval2Spec), "video": (VideoRewardScorer, VideoSpec),
    "videopickscore": (VideoPickScoreScorer, VideoPickScoreSpec),
}


def build_from_spec(name: str, config: Any = None, base_device: Optional[str] = None) -> Any:
    scorer_cls, spec_cls = REGISTRY[name]
    return scorer_cls(config=config if config is not None else spec_cls(), base_device=base_device)


__all__ = ["BaseRewardComponentSpec", "REGISTRY", "build_from_spec", *sorted({c.__name__ for pair in REGISTRY.values() for c in pair})]
