"""Device status words, read where the host synchronises anyway.

Kernels of this package never trap and never spin without a bound: a wait that runs out (an mbarrier in the tcgen05
GEMMs, a peer flag in the NVLink kernels) records a code in a device word, the kernel drains and returns, and its
output is garbage.  The host turns that word into an exception at the next step boundary — after a rollout batch,
inside the optimizer step — so training never continues on such output.

Sources: the per-device word of the GEMM / attention kernels (``_C.gemm_status``) and every live peer arena
(``PeerArena.check``), which register themselves here.
"""

from __future__ import annotations

import weakref
from typing import Any, Callable, List

from unirl_b200.ops import _ext


class DeviceKernelError(RuntimeError):
    """A kernel of this package gave up on a bounded wait; ``code`` names the kernel role (101-104 persistent GEMM, 121-126
    decode-sized GEMM, 141-149 attention, 300+ peer kernels)."""

    def __init__(self, code: int, where: str):
        super().__init__(f"device status word is {code} at {where}: a kernel's bounded wait ran out and its output is not valid")
        self.code, self.where = int(code), where


_checkers: List[Any] = []  # weak references to objects with a ``check()`` method


def register_checker(obj: Any) -> None:
    _checkers.append(weakref.ref(obj))


def check_device_status(where: str) -> None:
    """Raise ``DeviceKernelError`` / ``PeerCommError`` if any status word of the current device is non-zero (and clear it)."""
    import torch

    if not torch.cuda.is_available():
        return
    C = _ext.ext()
    if C is not None and hasattr(C, "gemm_status"):
        code = int(C.gemm_status(True))
        if code:
            raise DeviceKernelError(code, where)
    live = []
    for ref in _checkers:
        obj = ref()
        if obj is not None:
            live.append(ref)
            obj.check()
    _checkers[:] = live


__all__ = ["DeviceKernelError", "check_device_status", "register_checker"]
