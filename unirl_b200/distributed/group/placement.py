"""``placement`` scopes carve device slabs out of a pool; ``remote`` creates handles inside them.

``with placement(pool, fraction=0.5):`` claims half of the pool's unclaimed devices; a nested
scope carves the parent's slab.  Roles created in the same scope are co-located (they share
workers and therefore an address space — on one-process-per-GPU this is what lets the trainer
hand weights to the rollout engine by pointer).  Parity: ``unirl/distributed/group/placement.py``
(``Placement.assign`` ``:42-64``, scopes ``:73-141``, ``remote`` ``:144-169``).
"""

from __future__ import annotations

import contextlib
import threading
from typing import Any, Iterator, List, Optional, Sequence

_tls = threading.local()


class Placement:
    def __init__(self, pool: Any, devices: List[int], shared_workers: bool = True, parent: Optional["Placement"] = None):
        self.pool, self.devices, self.shared_workers, self.parent = pool, devices, shared_workers, parent
        self._carved = 0

    def carve(self, n: int) -> List[int]:
        if self._carved + n > len(self.devices):
            raise RuntimeError(f"placement slab of {len(self.devices)} devices cannot yield {n} more")
        got = self.devices[self._carved : self._carved + n]
        self._carved += n
        return got


def current_placement() -> Optional[Placement]:
    stack = getattr(_tls, "stack", None)
    return stack[-1] if stack else None


@contextlib.contextmanager
def placement(pool: Any, fraction: Optional[float] = None, num_devices: Optional[int] = None,
              devices: Optional[Sequence[int]] = None, shared_workers: bool = True) -> Iterator[Placement]:
    parent = current_placement()
    universe = len(parent.devices) if parent is not None else pool.num_devices
    if devices is not None:
        got = list(devices)
    else:
        n = num_devices if num_devices is not None else max(1, int(round(universe * (1.0 if fraction is None else fraction))))
        got = parent.carve(n) if parent is not None else pool.allocate(n)
    scope = Placement(pool, got, shared_workers, parent)
    if not hasattr(_tls, "stack"):
        _tls.stack = []
    _tls.stack.append(scope)
    try:
        yield scope
    finally:
        _tls.stack.pop()


def remote(role_cls: Any, role_name: Optional[str] = None, parallel: Optional[dict] = None, **init_kwargs: Any) -> Any:
    """Create a :class:`Handle` for ``role_cls`` on the devices of the enclosing placement scope."""
    scope = current_placement()
    if scope is None:
        raise RuntimeError("remote() must be called inside a `with placement(pool, ...)` block")
    return scope.pool.create_remote(role_cls, scope.devices, role_name=role_name, parallel=parallel, **init_kwargs)


def remote_cfg(cfg: Any, **extra: Any) -> Any:
    """``remote(**parse_cfg(cfg), **extra)`` — the recipe-driven spelling."""
    from unirl_b200.config.instantiate import parse_cfg

    return remote(**parse_cfg(cfg), **extra)


remote_hydra = remote_cfg

__all__ = ["Placement", "placement", "remote", "remote_cfg", "remote_hydra", "current_placement"]
