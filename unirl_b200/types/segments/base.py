"""``Segment`` — batched per-modality generation output; row ``k`` belongs to track sample ``k``.

Parity: ``unirl/types/segments/base.py:27-83``.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, ClassVar, Optional

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.types.conditions.base import Condition, Modality


class SegmentStatus(int, Enum):
    PENDING = 0
    COMPLETED = 1
    TRUNCATED = 2
    ABORTED = 3


@dataclass
class Segment(Batch):
    modality: ClassVar[Modality]
    status: Optional[torch.Tensor] = concat_field(default=None)

    def as_condition(self) -> Optional[Condition]:
        """Encoder-free promotion into the next stage's input (``None`` when not applicable)."""
        return None

    def as_condition_with(self, encoder: Callable[..., Any]) -> Condition:
        raise NotImplementedError(f"{type(self).__name__} has no encoder-mediated promotion")


__all__ = ["Segment", "SegmentStatus"]
