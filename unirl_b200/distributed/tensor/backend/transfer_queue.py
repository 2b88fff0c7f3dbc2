"""In-memory queue transport: puts are grouped by leading dimension into column sets.

The reference's GLOBAL transport rides on the external ``transfer_queue`` library with Mooncake
RDMA storage for multi-node jobs (``backend/transfer_queue/{runtime,transport,simple,mooncake}.py``).
A single NVSwitch box needs neither RDMA nor a storage actor, so this backend keeps the same
*semantics* — ``put_batch`` groups tensors that share a leading dimension into one record whose
columns are fetched together, zero-/one-dim tensors ride along reshaped, and buffers are
reclaimed per rollout — on top of the worker-local store.
"""

from __future__ import annotations

from typing import Any, Dict, List

import torch

from unirl_b200.distributed.tensor.transport import TensorMeta, WorkerLocalTransport


class QueueTransport(WorkerLocalTransport):
    def __init__(self, *a: Any, **k: Any):
        super().__init__(*a, **k)
        self._records: List[Dict[str, Any]] = []

    def put_batch(self, tensors: Dict[str, torch.Tensor]) -> Dict[str, TensorMeta]:
        by_rows: Dict[int, Dict[str, torch.Tensor]] = {}
        for name, t in tensors.items():
            by_rows.setdefault(int(t.shape[0]) if t.dim() else -1, {})[name] = t
        out: Dict[str, TensorMeta] = {}
        for rows, cols in by_rows.items():
            rec = {"rows": rows, "columns": {}}
            for name, t in cols.items():
                meta = self._put_scalar(t) if t.dim() == 0 else TensorMeta.from_refs([self.put(t)])
                rec["columns"][name] = meta
                out[name] = meta
            self._records.append(rec)
        return out

    def reclaim(self) -> int:
        """Drop every record written since the last reclaim (called once per rollout)."""
        n = 0
        for rec in self._records:
            for meta in rec["columns"].values():
                for r in meta.refs:
                    self.free(r)
                    n += 1
        self._records.clear()
        return n


# ---- configuration records of recipes written for the reference --------------------------------------------------------------
# ``transfer_queue: {_target_: …simple.SimpleBackend, num_units, unit_size}`` and the Mooncake variant describe the storage behind the
# GLOBAL queue plane.  On one NVSwitch box the queue lives in the workers' own memory whatever the record says; the records are kept so
# that such recipes load, and the Mooncake one says so once.
class SimpleBackend:
    def __init__(self, num_units: int = 16, unit_size: int = 1024, **_kw: Any):
        self.num_units, self.unit_size = int(num_units), int(unit_size)


class MooncakeZeroCopyConfig:
    def __init__(self, enable: bool = True, **kw: Any):
        self.enable, self.options = bool(enable), dict(kw)


class MooncakeBackend:
    def __init__(self, metadata_server: str = "", master_server_address: str = "", protocol: str = "rdma", zero_copy: Any = None, **kw: Any):
        import logging

        self.metadata_server, self.master_server_address, self.protocol, self.zero_copy, self.options = metadata_server, master_server_address, protocol, zero_copy, dict(kw)
        logging.getLogger(__name__).warning("transfer_queue: a Mooncake storage back end is configured; this build keeps the queue in the workers' memory "
                                            "(single NVSwitch domain), the RDMA settings are not used")


__all__ = ["QueueTransport", "SimpleBackend", "MooncakeBackend", "MooncakeZeroCopyConfig"]
