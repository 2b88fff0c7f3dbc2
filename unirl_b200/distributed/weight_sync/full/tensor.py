"""``TensorWeightSync`` — colocated sync: buckets of named tensors handed to the sibling engine in-process.

The reference serialises CUDA-IPC handles into a flattened bucket and POSTs them to the SGLang
server (``unirl/distributed/weight_sync/full/tensor.py:55-112``).  With one process per GPU the trainer
and the engine share an address space, so a "bucket" is a dict of tensor references; an engine that
aliases the trainer's replica (tp = 1) has nothing to copy at all.
"""

from __future__ import annotations

from typing import Dict

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.weight_sync.full.base import FullWeightSync


class TensorWeightSync(FullWeightSync):
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        if self._rollout is None:
            raise RuntimeError("TensorWeightSync needs a co-located `rollout` sibling")

        def run() -> int:
            n = 0
            for bucket, is_last in self._iter_buckets():
                n += int(self._rollout.update_weights_from_tensor(serialized_named_tensors=[dict(bucket)], load_format="named_dict",
                                                                   flush_cache=self._flush_cache and is_last, track_prefix=self._track_prefix) or 0)
            return n

        copied = self._timed(run)
        self.weight_version += 1
        return {"sync_ms": self.last_sync_ms, "tensors": float(copied), "weight_version": float(self.weight_version)}


__all__ = ["TensorWeightSync"]
