"""Fused multimodal condition: one interleaved token stream with per-position modality routing.

Used by unified AR+DiT models where text tokens, ViT embeddings and VAE latents share one
sequence.  Parity: ``unirl/types/conditions/fused_multimodal.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, List, Optional

import torch

from unirl_b200.distributed.tensor.batch import concat_field, shared_field
from unirl_b200.types.conditions.base import Condition, Modality


@dataclass
class FusedMultimodalCondition(Condition):
    modality: ClassVar[Modality] = Modality.MULTIMODAL

    input_ids: Optional[torch.Tensor] = concat_field(default=None)  # [B, L]
    attention_mask: Optional[torch.Tensor] = concat_field(default=None)  # [B, L]
    position_ids: Optional[torch.Tensor] = concat_field(default=None)
    image_embeds: Optional[torch.Tensor] = concat_field(default=None)  # [B, Nimg, D]
    image_mask: Optional[torch.Tensor] = concat_field(default=None)  # [B, L] bool: positions fed from image_embeds
    latent_mask: Optional[torch.Tensor] = concat_field(default=None)  # [B, L] bool: positions the DiT head generates
    extras: Dict[str, Any] = concat_field(default_factory=dict)
    layout: Optional[List[str]] = shared_field(default=None)


__all__ = ["FusedMultimodalCondition"]
