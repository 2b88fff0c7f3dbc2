"""LoRA sync payload: canonical tensors + PEFT config + optional checksums.  Parity: ``unirl/distributed/weight_sync/payload.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class LoraPayload:
    adapter_name: str
    tensors: Dict[str, torch.Tensor]
    peft_config: Dict[str, Any]
    version: int = 0
    checksums: Optional[Dict[str, str]] = None

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())


__all__ = ["LoraPayload"]
