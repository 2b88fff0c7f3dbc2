"""``Condition`` (encoded conditioning input) and the ``Modality`` tag.  Parity: ``unirl/types/conditions/base.py``."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import ClassVar

from unirl_b200.distributed.tensor.batch import Batch


class Modality(str, Enum):
    TEXT = "text"
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"
    MULTIMODAL = "multimodal"


@dataclass
class Condition(Batch):
    """Marker base; subclasses declare payload tensors and set ``modality``."""

    modality: ClassVar[Modality]


__all__ = ["Condition", "Modality"]
