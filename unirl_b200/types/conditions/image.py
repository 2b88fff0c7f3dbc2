"""Image conditions: VAE latents or ViT patch embeddings.  Parity: ``unirl/types/conditions/image.py``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, List, Optional, Tuple

import torch

from unirl_b200.distributed.tensor.batch import concat_field, shared_field
from unirl_b200.types.conditions.base import Condition, Modality


@dataclass
class ImageLatentCondition(Condition):
    modality: ClassVar[Modality] = Modality.IMAGE
    latents: Optional[torch.Tensor] = concat_field(default=None)


@dataclass
class ImageEmbedCondition(Condition):
    modality: ClassVar[Modality] = Modality.IMAGE
    embeds: Optional[torch.Tensor] = concat_field(default=None)
    attn_mask: Optional[torch.Tensor] = concat_field(default=None)
    spatial_shapes: Optional[List[Tuple[int, int]]] = shared_field(default=None)


__all__ = ["ImageLatentCondition", "ImageEmbedCondition"]
