"""``NCCLWeightSync`` — separate-slab sync by broadcast from trainer rank 0 to every engine rank.

This is the *baseline* transport for split placement (the product path is ``ReshardWeightSync``).
Handshake, driven by the controller: ``pick_master()`` → ``set_rollout_targets(engine worker ids)`` →
``connect()`` on the trainer side while the engine handle runs ``init_weights_update_group`` with the
same rank list (both sides build one process group from pool-global ranks).  ``sync()`` then, per
bucket, broadcasts each tensor from trainer rank 0 while the controller has the engine ranks
execute ``update_weights_from_distributed`` with the bucket's names/dtypes/shapes.
Parity: ``unirl/distributed/weight_sync/full/nccl.py:72-136`` (handshake), ``:142-181`` (sync).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.distributed.group.dispatch import Dispatch, Execute, distributed
from unirl_b200.distributed.weight_sync.full.base import FullWeightSync
from unirl_b200.utils.dtypes import dtype_name


class NCCLWeightSync(FullWeightSync):
    def __init__(self, *a, group_name: str = "weight_sync", **k) -> None:
        k.setdefault("bucket_size_mb", 512)
        super().__init__(*a, **k)
        self.group_name = group_name
        self._targets: List[int] = []
        self._sync_comm: Optional[Comm] = None

    @distributed(dispatch_mode=Dispatch.BROADCAST, execute_mode=Execute.RANK_ZERO)
    def pick_master(self) -> int:
        """Pool-global rank of the broadcasting trainer rank."""
        return int(self.comm.global_ranks[0]) if self.comm.active else int(self.dist_env.get("GLOBAL_RANK", 0))

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def set_rollout_targets(self, member_global_ranks: List[int], src_global_rank: int) -> None:
        self._targets, self._src = list(member_global_ranks), int(src_global_rank)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def connect(self) -> None:
        import torch.distributed as dist

        if self.rank_info.rank != 0:
            return
        ranks = sorted(set([self._src, *self._targets]))
        g = dist.new_group(ranks=ranks, use_local_synchronization=True) if dist.is_initialized() and len(ranks) > 1 else None
        self._sync_comm = Comm(g, ranks, self._src)
        self._src_local = ranks.index(self._src)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def bucket_plan(self) -> List[Dict[str, Any]]:
        """Names / dtypes / shapes per bucket, so the controller can post matching receives."""
        return [{"names": [n for n, _ in b], "dtypes": [dtype_name(t.dtype) for _, t in b], "shapes": [list(t.shape) for _, t in b]}
                for b, _ in self._iter_buckets()]

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def send_bucket(self, index: int) -> float:
        """Trainer side of one bucket: rank 0 broadcasts every tensor; other trainer ranks have nothing to do."""
        if self.rank_info.rank != 0:
            return 0.0

        def run() -> None:
            for i, (bucket, _last) in enumerate(self._iter_buckets()):
                if i != index:
                    continue
                for _n, t in bucket:
                    self._sync_comm.broadcast(t.contiguous(), src=self._src_local)

        self._timed(run)
        return self.last_sync_ms

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        raise RuntimeError("NCCLWeightSync.sync is controller-coordinated: use weight_sync.drive_nccl_sync(wsync, rollout)")

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def bump_version(self) -> int:
        self.weight_version += 1
        return self.weight_version


__all__ = ["NCCLWeightSync"]
