"""``IPCWeightSync`` — the bucketed staging-buffer protocol of the reference, collapsed to one process.

The reference pumps buckets through a 2 GiB CUDA-IPC staging buffer with ZMQ REQ/REP metadata while a
thread parks the receivers (``unirl/distributed/weight_sync/full/ipc.py:65-119``,
``rollout/engine/vllm_omni/weight_sync/bucketed_transfer.py:86-315``).  The staging discipline is kept —
tensors are packed into one reusable flat device buffer per dtype and the receiver unpacks views —
because it bounds peak memory for engines that do not alias the trainer's replica; the IPC handle
exchange and the sockets disappear.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.weight_sync.full.base import FullWeightSync


class IPCWeightSync(FullWeightSync):
    def __init__(self, *a, staging_size_mb: int = 2048, use_shm: bool = False, **k) -> None:
        """``use_shm`` is the reference's choice between a CUDA-IPC buffer and host shared memory for a receiver in another process
        (``unirl/distributed/weight_sync/full/ipc.py:46``); sender and receiver share one process here, so both values take the same
        device staging buffer and the field is only recorded."""
        super().__init__(*a, **k)
        self.use_shm = bool(use_shm)
        self._staging_bytes = int(staging_size_mb) * 1024 * 1024
        self._staging: Dict[torch.dtype, torch.Tensor] = {}

    def _stage(self, bucket: List[Tuple[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        by_dtype: Dict[torch.dtype, List[Tuple[str, torch.Tensor]]] = {}
        for n, t in bucket:
            by_dtype.setdefault(t.dtype, []).append((n, t))
        for dt, items in by_dtype.items():
            need = sum(t.numel() for _, t in items)
            buf = self._staging.get(dt)
            if buf is None or buf.numel() < need or buf.device != items[0][1].device:
                buf = torch.empty(max(need, self._staging_bytes // max(1, items[0][1].element_size()) // 8), dtype=dt, device=items[0][1].device)
                self._staging[dt] = buf
            off = 0
            for n, t in items:
                view = buf[off : off + t.numel()].view(t.shape)
                view.copy_(t)
                out[n] = view
                off += t.numel()
        return out

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        if self._rollout is None:
            raise RuntimeError("IPCWeightSync needs a co-located `rollout` sibling")

        def run() -> int:
            n = 0
            for bucket, is_last in self._iter_buckets():
                n += int(self._rollout.update_weights_from_tensor(serialized_named_tensors=[self._stage(bucket)], load_format="staged",
                                                                   flush_cache=self._flush_cache and is_last, track_prefix=self._track_prefix) or 0)
            return n

        copied = self._timed(run)
        self.weight_version += 1
        return {"sync_ms": self.last_sync_ms, "tensors": float(copied), "weight_version": float(self.weight_version)}


__all__ = ["IPCWeightSync"]
