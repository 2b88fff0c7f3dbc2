"""Controller-side choreography for weight-sync transports that span two device slabs."""

from __future__ import annotations

from typing import Any, Dict


def connect_nccl_sync(wsync: Any, rollout: Any) -> None:
    """One-time handshake: both sides build the broadcast group from pool-global ranks."""
    pool = wsync.pool
    src = wsync.devices[0]
    targets = list(rollout.devices)
    wsync.set_rollout_targets(targets, src)
    c1, x1 = wsync.prepare("connect")
    c2, x2 = rollout.prepare("init_weights_update_group", src_global_rank=src, member_global_ranks=targets, group_name=_group_name(wsync))
    pool.run_many([c1, c2])


def _group_name(wsync: Any) -> str:
    return "weight_sync"


def drive_nccl_sync(wsync: Any, rollout: Any) -> Dict[str, float]:
    """Per bucket: trainer rank 0 broadcasts while every engine rank receives and loads."""
    pool = wsync.pool
    plan = wsync.bucket_plan()[0]
    total_ms = 0.0
    for i, b in enumerate(plan):
        c1, x1 = wsync.prepare("send_bucket", i)
        c2, x2 = rollout.prepare("update_weights_from_distributed", names=b["names"], dtypes=b["dtypes"], shapes=b["shapes"], group_name=_group_name(wsync))
        r1, _r2 = pool.run_many([c1, c2])
        total_ms += float(r1[0] or 0.0)
    version = wsync.bump_version()[0]
    return {"sync_ms": total_ms, "buckets": float(len(plan)), "weight_version": float(version)}


__all__ = ["connect_nccl_sync", "drive_nccl_sync"]
