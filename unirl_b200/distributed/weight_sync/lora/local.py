"""``LocalLoraWeightSync`` — colocated: every rank hands its adapter tensors to the sibling engine.
Parity: ``unirl/distributed/weight_sync/lora/local.py:51-88``."""

from __future__ import annotations

import time
from typing import Dict

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.weight_sync.lora.base import LoraWeightSyncBase


class LocalLoraWeightSync(LoraWeightSyncBase):
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        if self._rollout is None:
            raise RuntimeError("LocalLoraWeightSync needs a co-located `rollout` sibling")
        t0 = time.perf_counter()
        payload = self._extract()
        self._rollout.set_lora_from_tensors(payload.adapter_name, payload.tensors, peft_config=payload.peft_config)
        self.weight_version = payload.version
        self.last_sync_ms = (time.perf_counter() - t0) * 1e3
        return {"sync_ms": self.last_sync_ms, "tensors": float(len(payload.tensors)), "bytes": float(payload.nbytes()),
                "weight_version": float(self.weight_version)}


__all__ = ["LocalLoraWeightSync"]
