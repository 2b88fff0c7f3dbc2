"""``RemoteLoraWeightSync`` — cross-slab LoRA sync: ``extract()`` on the trainer ranks (rank 0 keeps the
payload), ``push()`` returns it to the controller which forwards it to every engine worker; ``sync_remote``
(controller helper) = both + optional checksum verification.  Parity:
``unirl/distributed/weight_sync/lora/remote.py:67-149`` (extract / push / sync), ``:153-178`` (verify).
"""

from __future__ import annotations

import time
from typing import Any, Dict, Optional

from unirl_b200.distributed.group.dispatch import Dispatch, Execute, distributed
from unirl_b200.distributed.weight_sync.lora.base import LoraWeightSyncBase
from unirl_b200.distributed.weight_sync.payload import LoraPayload
from unirl_b200.distributed.utils import Broadcast


class RemoteLoraWeightSync(LoraWeightSyncBase):
    def __init__(self, *a: Any, copy: bool = False, **k: Any) -> None:
        super().__init__(*a, **k)
        self._copy = bool(copy)
        self._cached: Optional[LoraPayload] = None

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def extract(self) -> int:
        payload = self._extract()
        if self.rank_info.rank == 0:
            self._cached = payload
        return len(payload.tensors)

    @distributed(dispatch_mode=Dispatch.BROADCAST, execute_mode=Execute.RANK_ZERO)
    def push(self) -> Dict[str, Any]:
        """Hand the cached payload to the controller (plain CPU tensors inside a dict travel by value)."""
        if self._cached is None:
            raise RuntimeError("RemoteLoraWeightSync.push before extract")
        p = self._cached
        self.weight_version = p.version
        out = {"adapter_name": p.adapter_name, "tensors": {k: (v.clone() if self._copy else v) for k, v in p.tensors.items()},
               "peft_config": p.peft_config, "version": p.version,
               "checksum": sorted(self._checksum(p).items()) if self._verify else None}
        return _Opaque(out)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        raise RuntimeError("RemoteLoraWeightSync.sync is controller-coordinated: use sync_remote_lora(wsync, rollout)")


class _Opaque:
    """Wrapper that hides tensors from the transport's dehydration (adapter payloads are small and go by value)."""

    def __init__(self, value: Any):
        self.value = value


def sync_remote_lora(wsync: Any, rollout: Any, verify: bool = False) -> Dict[str, float]:
    t0 = time.perf_counter()
    wsync.extract()
    payload = wsync.push()[0].value
    rollout.set_lora_from_tensors(Broadcast(payload["adapter_name"]), Broadcast(_Opaque(payload["tensors"])), peft_config=Broadcast(payload["peft_config"]))
    if verify and payload["checksum"] is not None:
        theirs = rollout.compute_lora_checksums(Broadcast(payload["adapter_name"]))
        for r, c in enumerate(theirs):
            if sorted(c.items()) != payload["checksum"]:
                raise RuntimeError(f"LoRA checksum mismatch on engine rank {r}")
    return {"sync_ms": (time.perf_counter() - t0) * 1e3, "tensors": float(len(payload["tensors"])), "weight_version": float(payload["version"])}


__all__ = ["RemoteLoraWeightSync", "sync_remote_lora"]
