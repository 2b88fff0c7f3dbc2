"""Loader for the in-tree native extension ``unirl_b200/_C*.so`` (built by ``unirl_b200.build``)."""

from __future__ import annotations

import importlib
import os
import threading
from typing import Any, Optional

_lock = threading.Lock()
_mod: Optional[Any] = None
_err: Optional[BaseException] = None
_launches = 0


def ext() -> Optional[Any]:
    """The native module, or ``None`` when it is not built (CPU-only checkout)."""
    global _mod, _err
    if _mod is None and _err is None:
        with _lock:
            if _mod is None and _err is None:
                try:
                    import torch  # noqa: F401  (the extension links against libtorch)

                    _mod = importlib.import_module("unirl_b200._C")
                    if os.environ.get("UNIRL_B200_PDL", "1") == "0" and hasattr(_mod, "set_pdl"):
                        _mod.set_pdl(False)  # decode-sized kernels then keep plain stream order
                except BaseException as e:  # noqa: BLE001
                    _err = e
    return _mod


def have_ext() -> bool:
    return ext() is not None


def require_ext() -> Any:
    m = ext()
    if m is None:
        raise RuntimeError("unirl_b200._C is not built or failed to load; run `python -m unirl_b200.build` "
                           f"(CUDA tensors are never served by an eager fallback). Cause: {_err!r}")
    return m


def use_native(*tensors: Any) -> bool:
    """True when the op must run on the native kernel (any CUDA tensor)."""
    if os.environ.get("UNIRL_B200_FORCE_REFERENCE") == "1":
        return False
    return any(getattr(t, "is_cuda", False) for t in tensors)


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launch_count() -> int:
    """Number of native kernel launches issued through the op layer since import (bench bookkeeping)."""
    return _launches


__all__ = ["ext", "have_ext", "require_ext", "use_native", "count_launch", "launch_count"]
