"""Tracing and profiling switches: NVTX ranges around the loop phases, a capture window for external profilers, and per-step
roofline fractions of the two phases that dominate a step.

* ``nvtx_range(name)`` / ``set_nvtx(True)``: phase names become NVTX ranges (visible in Nsight Systems / Compute); off by default, so
  the hot loop pays nothing.
* ``ProfileWindow``: ``profile.enabled=true profile.start_step=S profile.num_steps=N`` (or ``--profile`` on an entry point, or
  ``UNIRL_B200_PROFILE=S:N``) brackets steps ``S .. S+N-1`` with ``cudaProfilerStart/Stop`` (use with
  ``ncu --profile-from-start off`` or ``nsys --capture-range cudaProfilerApi``) and, when ``profile.trace_dir`` is set, writes a
  ``torch.profiler`` Chrome trace of those steps.
* ``roofline_metrics``: ``kernel/train_tflops``, ``kernel/train_roofline_frac``, ``kernel/decode_gbs``, ``kernel/decode_roofline_frac``
  from the phase times of a step, the model's parameter count and the tokens it produced, against the measured peaks
  (``MEASURED_PEAKS.json`` at the repository root; the documented fallback otherwise).

The reference times phases on the host only (``unirl/utils/wandb_logger.py:43-142``); these are the device-side additions.
"""

from __future__ import annotations

import contextlib
import json
import os
from typing import Any, Dict, Iterator, Optional

import torch

_NVTX = os.environ.get("UNIRL_B200_NVTX", "0") == "1"


def set_nvtx(on: bool) -> None:
    global _NVTX
    _NVTX = bool(on)


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def measured_peaks() -> Dict[str, Any]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "kind": "of measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "kind": "of fallback"}


def roofline_metrics(*, n_params: int, train_tokens: int, train_ms: float, decode_tokens: int, decode_steps: int, rollout_ms: float,
                     kv_bytes_per_token: int = 0, mean_context: float = 0.0, batch: int = 0, weight_bytes: Optional[int] = None) -> Dict[str, float]:
    """Roofline fractions of a step.  Training: 6·N·tokens model FLOPs (forward + backward, attention excluded) over the phase time,
    against the sustained GEMM peak.  Decode: every step streams the weights once plus the KV cache of every live sequence."""
    pk = measured_peaks()
    out: Dict[str, float] = {}
    if train_ms > 0 and train_tokens > 0:
        tf = 6.0 * n_params * train_tokens / (train_ms * 1e-3) / 1e12
        out["kernel/train_tflops"] = tf
        out["kernel/train_roofline_frac"] = tf / pk["tflops_sustained"]
    if rollout_ms > 0 and decode_steps > 0:
        wb = weight_bytes if weight_bytes is not None else 2 * n_params
        total = decode_steps * (wb + kv_bytes_per_token * mean_context * batch)
        gbs = total / (rollout_ms * 1e-3) / 1e9
        out["kernel/decode_gbs"] = gbs
        out["kernel/decode_roofline_frac"] = gbs / pk["hbm_gbs"]
    return out


class ProfileWindow:
    """Brackets a window of steps for an external profiler and / or records a ``torch.profiler`` trace of it."""

    def __init__(self, enabled: bool = False, start_step: int = 3, num_steps: int = 1, trace_dir: Optional[str] = None, nvtx: bool = True):
        env = os.environ.get("UNIRL_B200_PROFILE")
        if env:
            enabled = True
            a, _, b = env.partition(":")
            start_step, num_steps = int(a or 3), int(b or 1)
        self.enabled, self.start, self.stop = bool(enabled), int(start_step), int(start_step) + int(num_steps)
        self.trace_dir = trace_dir
        self._prof: Any = None
        self._active = False
        if self.enabled and nvtx:
            set_nvtx(True)

    @classmethod
    def from_cfg(cls, cfg: Any) -> "ProfileWindow":
        if cfg is None:
            return cls()
        get = cfg.get if hasattr(cfg, "get") else lambda k, d=None: getattr(cfg, k, d)
        return cls(bool(get("enabled", False)), int(get("start_step", 3)), int(get("num_steps", 1)), get("trace_dir", None), bool(get("nvtx", True)))

    def step_begin(self, step: int) -> None:
        if not self.enabled or self._active or not (self.start <= step < self.stop):
            return
        self._active = True
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
        if self.trace_dir:
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            self._prof = torch.profiler.profile(activities=acts)
            self._prof.__enter__()

    def step_end(self, step: int) -> None:
        if not self._active or step + 1 < self.stop:
            return
        self._active = False
        if self._prof is not None:
            self._prof.__exit__(None, None, None)
            os.makedirs(self.trace_dir, exist_ok=True)
            self._prof.export_chrome_trace(os.path.join(self.trace_dir, f"trace_steps_{self.start}_{self.stop - 1}.json"))
            self._prof = None
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()


__all__ = ["nvtx_range", "set_nvtx", "nvtx_enabled", "ProfileWindow", "roofline_metrics", "measured_peaks"]
