"""Text conditions: encoder hidden states (``TextEmbedCondition``) or token ids (``TextTokenCondition``).

Both pad the sequence axis to the longest member before concatenation, because DP shards encode /
right-pad to their own in-shard maximum.  Parity: ``unirl/types/conditions/text.py:38-129``.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import ClassVar, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.types.conditions.base import Condition, Modality


def pad_seq_axis(t: Optional[torch.Tensor], target: int) -> Optional[torch.Tensor]:
    if t is None or t.dim() < 2 or t.shape[1] == target:
        return t
    if t.shape[1] > target:
        raise ValueError(f"cannot pad sequence axis {t.shape[1]} down to {target}")
    pad = [0, 0] * (t.dim() - 2) + [0, target - t.shape[1]]
    return F.pad(t, pad, value=0)


class _SeqPadConcat:
    """Mixin: ``concat`` that zero-pads the named ``[B, T, …]`` fields to a common ``T``."""

    _seq_fields: ClassVar[Tuple[str, ...]] = ()

    @classmethod
    def concat(cls, items: Sequence["Batch"]):
        items = list(items)
        lens = {int(getattr(it, n).shape[1]) for it in items for n in cls._seq_fields
                if isinstance(getattr(it, n), torch.Tensor) and getattr(it, n).dim() >= 2}
        if len(items) > 1 and len(lens) > 1:
            target = max(lens)
            items = [it.replace(**{n: pad_seq_axis(getattr(it, n), target) for n in cls._seq_fields}) for it in items]
        return Batch.concat.__func__(cls, items)


@dataclass
class TextEmbedCondition(_SeqPadConcat, Condition):
    modality: ClassVar[Modality] = Modality.TEXT
    _seq_fields: ClassVar[Tuple[str, ...]] = ("embeds", "attn_mask")

    embeds: Optional[torch.Tensor] = concat_field(default=None)
    pooled: Optional[torch.Tensor] = concat_field(default=None)
    attn_mask: Optional[torch.Tensor] = concat_field(default=None)


@dataclass
class TextTokenCondition(_SeqPadConcat, Condition):
    modality: ClassVar[Modality] = Modality.TEXT
    _seq_fields: ClassVar[Tuple[str, ...]] = ("input_ids", "attention_mask")

    input_ids: Optional[torch.Tensor] = concat_field(default=None)
    attention_mask: Optional[torch.Tensor] = concat_field(default=None)


__all__ = ["TextEmbedCondition", "TextTokenCondition", "pad_seq_axis"]
