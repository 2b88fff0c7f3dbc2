"""Shared LoRA-sync logic: extract canonical adapter tensors + PEFT config, optional checksum verify.

``_extract`` walks the adapters of the trainer's module (resident on every rank — no gather needed),
emits ``<track_prefix><module>.lora_{A,B}.weight`` on CPU with a bf16/fp16/fp32 dtype guard, and the
PEFT config dict the receiving engine needs.  Verification compares order-free multisets of
SHA-256/16 fingerprints with ``lora_B`` scaled by ``alpha / r``.  Parity:
``unirl/distributed/weight_sync/lora/base.py:29-129``.
"""

from __future__ import annotations

import time
from typing import Any, Dict, Optional

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.distributed.weight_sync.checksum import lora_checksum_multiset
from unirl_b200.distributed.weight_sync.payload import LoraPayload
from unirl_b200.train.inject import peft_config_dict
from unirl_b200.utils.peft_merge import extract_lora_tensors


class LoraWeightSyncBase(Remote):
    def __init__(self, *, backend: Any, rollout: Any = None, adapter_name: str = "default", track_prefix: str = "", verify: bool = False,
                 param_prefix: str = "") -> None:
        """``param_prefix``: accepted for recipes written for the reference, where it names the engine-side module that holds the adapters
        (``transformer.``); the native engines address their transformer directly, so the adapter keys travel without it."""
        super().__init__()
        self._param_prefix = str(param_prefix or "")
        self._backend, self._rollout = backend, rollout
        self.adapter_name, self._track_prefix, self._verify = adapter_name, str(track_prefix or ""), bool(verify)
        self.weight_version = 0
        self.last_sync_ms = 0.0

    def _extract(self) -> LoraPayload:
        meta = getattr(self._backend, "_lora_meta", None)
        if meta is None:
            raise RuntimeError("LoRA weight sync needs a backend built with lora_cfg / ema_lora_cfg")
        tensors = extract_lora_tensors(self._backend.model, self.adapter_name, prefix=self._track_prefix)
        return LoraPayload(self.adapter_name, tensors, peft_config_dict(meta["rank"], meta["alpha"], meta["target_modules"]), self.weight_version + 1)

    def _checksum(self, payload: LoraPayload):
        return lora_checksum_multiset(payload.tensors, payload.peft_config["lora_alpha"], payload.peft_config["r"])

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def get_weight_version(self) -> int:
        return self.weight_version


__all__ = ["LoraWeightSyncBase"]
