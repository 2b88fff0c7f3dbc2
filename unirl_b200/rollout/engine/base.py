"""Rollout-engine contract.

``generate(req)`` plus the life-cycle and weight-receive surface the trainers and weight-sync
handlers drive: ``sleep`` / ``wake_up`` (release / re-acquire HBM by region), ``health_check``,
``get_memory_info``, and the receive methods (``update_weights_from_tensor`` / ``..._from_distributed`` /
``..._from_ipc`` / ``set_lora_from_tensors`` / process-group management).  Native engines implement the
receive side as writes into their own (TP-sharded) weight buffers.  Parity:
``unirl/rollout/engine/base.py:45-192``, ``__init__.py:14-51`` (``chunked_engine_generate_req``).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp


class BaseRolloutEngine(Remote, ABC):
    _component_name = "base"

    @abstractmethod
    def generate(self, req: RolloutReq) -> RolloutResp: ...

    def shutdown(self) -> None:
        pass

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sleep(self) -> None:
        """Release rollout-only memory (KV cache, graphs). Default: nothing to release."""

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def wake_up(self) -> None:
        """Re-acquire what ``sleep`` released."""

    def onload_weights(self, *, track_prefix: str = "") -> None:
        self.wake_up()

    @property
    def is_offloaded(self) -> bool:
        return False

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def health_check(self) -> bool:
        return True

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def get_memory_info(self) -> Dict[str, float]:
        if not torch.cuda.is_available():
            return {}
        return {"allocated_gb": torch.cuda.memory_allocated() / 1e9, "cached_gb": torch.cuda.memory_reserved() / 1e9}

    # ---- weight receive surface (engines override what they support) ----------------------------------
    def update_weights_from_ipc(self, *, peft_config: Optional[dict] = None, base_sync_done: bool = False, use_shm: bool = False,
                                track_prefix: str = "") -> None:
        raise NotImplementedError

    def init_weights_update_group(self, *, master_address: str, master_port: int, rank_offset: int, world_size: int, group_name: str,
                                  backend: str = "nccl", track_prefix: str = "") -> None:
        raise NotImplementedError

    def update_weights_from_distributed(self, *, names: List[str], dtypes: List[str], shapes: List[List[int]], group_name: str,
                                        target_modules: Optional[List[str]] = None, flush_cache: bool = True, track_prefix: str = "") -> None:
        raise NotImplementedError

    def destroy_weights_update_group(self, *, group_name: str, track_prefix: str = "") -> None:
        raise NotImplementedError

    def set_lora_from_tensors(self, adapter_name: str, lora_tensors: Dict[str, torch.Tensor], *, peft_config: Optional[dict] = None) -> None:
        raise NotImplementedError

    def update_weights_from_tensor(self, *, serialized_named_tensors: List[Any], target_modules: Optional[List[str]] = None,
                                   load_format: Optional[str] = None, flush_cache: bool = True, track_prefix: str = "") -> None:
        raise NotImplementedError


def chunked_engine_generate_req(req: RolloutReq, fn: Callable[[RolloutReq], RolloutResp], chunk: Optional[int]) -> RolloutResp:
    """Run ``fn`` over ``req`` in slices of ``chunk`` samples and concatenate the responses."""
    n = req.batch_size
    if not chunk or n <= chunk:
        return fn(req)
    return RolloutResp.concat([fn(req.slice(s, min(s + chunk, n))) for s in range(0, n, chunk)])


__all__ = ["BaseRolloutEngine", "chunked_engine_generate_req"]
