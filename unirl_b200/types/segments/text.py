"""``TextSegment`` — ragged token rollouts packed along dim 0 (``cu_seqlens`` managed by ``Batch``).

The packed layout is consumed as-is by the varlen attention and fused log-prob kernels: no
re-padding on the replay path.  Parity: ``unirl/types/segments/text.py:32-57``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, ClassVar, Optional

import torch

from unirl_b200.distributed.tensor.batch import packed_field
from unirl_b200.types.conditions.base import Condition, Modality
from unirl_b200.types.conditions.text import TextEmbedCondition
from unirl_b200.types.segments.base import Segment


@dataclass
class TextSegment(Segment):
    modality: ClassVar[Modality] = Modality.TEXT

    tokens: Optional[torch.Tensor] = packed_field(default=None)
    log_probs: Optional[torch.Tensor] = packed_field(default=None)
    loss_mask: Optional[torch.Tensor] = packed_field(default=None)

    def as_condition_with(self, encoder: Callable[..., Any]) -> Condition:
        if self.tokens is None:
            raise ValueError("TextSegment has no tokens to re-embed")
        out = encoder(self.tokens)
        return TextEmbedCondition(embeds=getattr(out, "embeds", out))


__all__ = ["TextSegment"]
