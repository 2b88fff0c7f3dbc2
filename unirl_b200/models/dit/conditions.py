"""Typed conditions of a DiT diffusion stage: positive text, optional negative text (CFG) and optional image latents
(image-to-video first frame / edit source).  Parity: ``unirl/models/sd3/conditions.py``, ``unirl/models/wan21/conditions.py``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.types.conditions import Condition, ImageEmbedCondition, ImageLatentCondition, TextEmbedCondition


@dataclass
class DiTConditions(Batch):
    text: Optional[TextEmbedCondition] = concat_field(default=None)
    negative_text: Optional[TextEmbedCondition] = concat_field(default=None)
    image: Optional[ImageLatentCondition] = concat_field(default=None)
    image_embed: Optional[ImageEmbedCondition] = concat_field(default=None)  # image-encoder tokens (WAN 2.1 image-to-video)

    @classmethod
    def from_dict(cls, d: Dict[str, Condition]) -> "DiTConditions":
        t = d.get("text")
        if not isinstance(t, TextEmbedCondition):
            raise TypeError(f"DiTConditions: d['text'] must be a TextEmbedCondition, got {type(t).__name__}")
        return cls(text=t, negative_text=d.get("negative_text"), image=d.get("image"), image_embed=d.get("image_embed"))

    def to_dict(self) -> Dict[str, Condition]:
        out: Dict[str, Condition] = {"text": self.text}
        if self.negative_text is not None:
            out["negative_text"] = self.negative_text
        if self.image is not None:
            out["image"] = self.image
        if self.image_embed is not None:
            out["image_embed"] = self.image_embed
        return out


__all__ = ["DiTConditions"]
