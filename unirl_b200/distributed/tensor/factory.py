"""``build_transport`` — pick the tensor-transport backend for a worker.

``colocate_store`` and ``gpu_store`` both resolve to the in-process refcounted store (one
process per GPU makes the reference's cross-process CUDA-IPC store, ``backend/gpu_store``, a
pointer hand-off); ``transfer_queue`` resolves to the in-memory queue backend.  Parity:
``unirl/distributed/tensor/factory.py:17-63``.
"""

from __future__ import annotations

from typing import Any, Optional

import torch


def build_transport(kind: str, worker_id: int, device: Any, comm: Optional[Any] = None, **_ignored: Any):
    from unirl_b200.distributed.tensor.backend.transfer_queue import QueueTransport
    from unirl_b200.distributed.tensor.transport import WorkerLocalTransport

    if kind in ("colocate_store", "gpu_store", "local"):
        return WorkerLocalTransport(worker_id, torch.device(device), comm)
    if kind in ("transfer_queue", "queue"):
        return QueueTransport(worker_id, torch.device(device), comm)
    raise ValueError(f"unknown tensor transport '{kind}'")


__all__ = ["build_transport"]
