"""``RankInfo`` and ``Remote`` — what a worker-side role knows about itself.

Every loop stage (rollout engine, train stack, reward service, weight sync, algorithm, bundle,
pipeline) derives from :class:`Remote`; that is the only coupling from model/loop code into the
runtime.  Parity: ``unirl/distributed/group/remote.py:21-61`` (RankInfo), ``:64-119`` (Remote),
``:123-188`` (auto-backward RPC).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.distributed.group.dispatch import Dispatch, distributed


@dataclass
class RankInfo:
    rank: int = 0
    world_size: int = 1
    dp_rank: int = 0
    dp_size: int = 1
    tp_rank: int = 0
    tp_size: int = 1
    pp_rank: int = 0
    pp_size: int = 1
    sp_rank: int = 0
    sp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1

    @property
    def is_pipeline_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @property
    def is_dp_rank_zero(self) -> bool:
        return self.dp_rank == 0

    def __repr__(self) -> str:
        bits = [f"rank={self.rank}/{self.world_size}"]
        for ax in ("dp", "tp", "pp", "sp", "ep"):
            n = getattr(self, f"{ax}_size")
            if n > 1:
                bits.append(f"{ax}={getattr(self, ax + '_rank')}/{n}")
        return "RankInfo(" + ", ".join(bits) + ")"


def make_rank_infos(world: int, tp: int = 1, sp: int = 1, pp: int = 1, ep: int = 1) -> List[RankInfo]:
    """Row-major ``(dp, pp, sp, tp)`` layout: tp is the fastest axis so TP peers are NVLink neighbours."""
    inner = tp * sp * pp
    if world % inner:
        raise ValueError(f"world={world} not divisible by tp*sp*pp={inner}")
    dp = world // inner
    out = []
    for r in range(world):
        tp_r = r % tp
        sp_r = (r // tp) % sp
        pp_r = (r // (tp * sp)) % pp
        dp_r = r // inner
        out.append(RankInfo(r, world, dp_r, dp, tp_r, tp, pp_r, pp, sp_r, sp, ep_rank=r % ep if ep > 1 else 0, ep_size=ep))
    return out


class Remote:
    """Base class of every worker-side role.

    Attributes injected by ``Worker.add_remote`` before ``__init__`` returns control to user code
    via :meth:`setup`: ``transport``, ``device``, ``rank_info``, ``dist_env``, ``comm`` (the role's
    process group wrapper) and a sibling lookup for co-located roles.
    """

    def __init__(self) -> None:
        self.transport = None
        self.device: Optional[str] = None
        self.rank_info: RankInfo = RankInfo()
        self.dist_env: Dict[str, str] = {}
        self.comm: Comm = Comm.solo()
        self._get_sibling: Optional[Callable[[str], "Remote"]] = None
        self._grad_inputs: Dict[str, List[torch.Tensor]] = {}
        self._grad_outputs: Dict[str, List[torch.Tensor]] = {}

    def _ensure_base(self) -> None:
        if not hasattr(self, "_grad_inputs"):
            Remote.__init__(self)

    def setup(self, transport: Any, device: str, rank_info: RankInfo, dist_env: Optional[Dict[str, str]] = None,
              get_sibling: Optional[Callable[[str], "Remote"]] = None, comm: Optional[Comm] = None) -> None:
        self._ensure_base()
        self.transport = transport
        self.device = device
        self.rank_info = rank_info
        self.dist_env = dict(dist_env or {})
        self._get_sibling = get_sibling
        self.comm = comm or Comm.solo()
        if self.dist_env:
            os.environ.update({k: str(v) for k, v in self.dist_env.items()})

    def get_sibling(self, name: str) -> "Remote":
        if self._get_sibling is None:
            raise RuntimeError("no sibling lookup available on this role")
        return self._get_sibling(name)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def initialize(self, *args: Any, **kwargs: Any) -> None:
        """Post-construction hook (load weights, build sub-groups)."""

    # ---- RPC autograd ---------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def _auto_backward(self, call_id: str, out_grads: tuple, in_grads: tuple) -> tuple:
        """Backward half of a recorded forward RPC: seeds saved outputs with ``out_grads`` and
        returns the accumulated ``.grad`` of every saved input (``None`` where there is none)."""
        self._ensure_base()
        outs = self._grad_outputs.pop(call_id, [])
        ins = self._grad_inputs.pop(call_id, [])
        for t, g in zip(ins, in_grads):
            if g is not None:
                t.grad = g
        pairs = [(t, g) for t, g in zip(outs, out_grads) if g is not None and (t.requires_grad or t.grad_fn is not None)]
        if pairs:
            torch.autograd.backward([t for t, _ in pairs], [g for _, g in pairs])
        return tuple(t.grad for t in ins)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def _cleanup_all_grads(self) -> None:
        self._ensure_base()
        self._grad_inputs.clear()
        self._grad_outputs.clear()


__all__ = ["RankInfo", "Remote", "make_rank_infos"]
