"""σ schedules for flow matching: pure math, a per-model policy object, and request glue.

Static shift ``σ = s·t / (1 + (s−1)·t)`` over ``linspace(1, 0, T+1)``; dynamic shift maps the base
grid ``linspace(1, 1/T, T)`` through ``e^μ / (e^μ + (1/t − 1))`` (or the linear variant) and appends
the terminal 0, with μ interpolated linearly in the image token count.  Parity:
``unirl/sde/runtime.py:71-130`` (math), ``:192-428`` (policy), ``:436-462`` (``ensure_req_sigmas``).
The reference delegates the dynamic branch to diffusers; it is restated here because diffusers
is not a dependency.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Optional

import torch

from unirl_b200.types.sampling import get_diffusion_params


def get_sigma_schedule(num_steps: int, shift: float = 3.0, device: Optional[Any] = None, *, mu: Optional[float] = None,
                       time_shift_type: str = "exponential") -> torch.Tensor:
    if mu is None:
        t = torch.linspace(1.0, 0.0, num_steps + 1)
        sig = (shift * t) / (1 + (shift - 1) * t)
    else:
        t = torch.linspace(1.0, 1.0 / num_steps, num_steps, dtype=torch.float64)
        num = math.exp(mu) if time_shift_type == "exponential" else float(mu)
        sig = torch.cat([(num / (num + (1.0 / t - 1.0))).float(), torch.zeros(1)])
    return sig.to(device) if device is not None else sig


def calculate_dynamic_mu(image_seq_len: int, base_seq_len: int = 256, max_seq_len: int = 4096, base_shift: float = 0.5,
                         max_shift: float = 1.15) -> float:
    m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
    return image_seq_len * m + (base_shift - m * base_seq_len)


def _read_json(path: str) -> Optional[dict]:
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


@dataclass
class FlowMatchSchedulePolicy:
    """Model-owned schedule policy: light, picklable, no weights needed."""

    shift: float = 3.0
    use_dynamic_shifting: bool = False
    base_shift: float = 0.5
    max_shift: float = 1.15
    base_image_seq_len: int = 256
    max_image_seq_len: int = 4096
    time_shift_type: str = "exponential"
    vae_scale_factor: int = 8
    patch_size: int = 2

    def compute_mu(self, image_seq_len: int, num_inference_steps: int) -> float:
        """Per-model override point (e.g. an empirical μ that also depends on the step count)."""
        return calculate_dynamic_mu(image_seq_len, self.base_image_seq_len, self.max_image_seq_len, self.base_shift, self.max_shift)

    def image_seq_len(self, height: int, width: int) -> int:
        return (int(height) // self.vae_scale_factor // self.patch_size) * (int(width) // self.vae_scale_factor // self.patch_size)

    def compute_sigma(self, *, num_inference_steps: int, height: int, width: int, device: Optional[Any] = None) -> torch.Tensor:
        if not self.use_dynamic_shifting:
            return get_sigma_schedule(num_inference_steps, self.shift, device)
        mu = self.compute_mu(self.image_seq_len(height, width), num_inference_steps)
        return get_sigma_schedule(num_inference_steps, self.shift, device, mu=mu, time_shift_type=self.time_shift_type)

    @classmethod
    def static_only(cls, shift: float) -> "FlowMatchSchedulePolicy":
        return cls(shift=float(shift), use_dynamic_shifting=False)

    @classmethod
    def from_pretrained(cls, path: Optional[str], shift: Optional[float] = None, **overrides: Any) -> "FlowMatchSchedulePolicy":
        """Read ``scheduler/scheduler_config.json``, ``vae/config.json`` and ``transformer/config.json`` when present."""
        kw: dict = {}
        if path and os.path.isdir(path):
            sch = _read_json(os.path.join(path, "scheduler", "scheduler_config.json")) or {}
            for k in ("shift", "use_dynamic_shifting", "base_shift", "max_shift", "base_image_seq_len", "max_image_seq_len", "time_shift_type"):
                if sch.get(k) is not None:
                    kw[k] = sch[k]
            vae = _read_json(os.path.join(path, "vae", "config.json")) or {}
            boc = vae.get("block_out_channels")
            if isinstance(boc, (list, tuple)) and boc:
                kw["vae_scale_factor"] = 2 ** (len(boc) - 1)
            tr = _read_json(os.path.join(path, "transformer", "config.json")) or {}
            ps = tr.get("patch_size")
            if isinstance(ps, (list, tuple)):
                ps = ps[-1]
            if ps:
                kw["patch_size"] = int(ps)
        if shift is not None:
            kw["shift"] = float(shift)
        kw.update({k: v for k, v in overrides.items() if v is not None})
        return cls(**kw)


def ensure_req_sigmas(req: Any, policy: FlowMatchSchedulePolicy) -> None:
    """Pin the schedule on ``req.sigmas`` once; later callers (engines) find it set and reuse it."""
    if req.sigmas is not None:
        return
    d = get_diffusion_params(req.sampling_params)
    if d is None:
        raise ValueError("ensure_req_sigmas: request carries no diffusion sampling params")
    req.sigmas = policy.compute_sigma(num_inference_steps=int(d.num_inference_steps), height=int(d.height), width=int(d.width))


__all__ = ["get_sigma_schedule", "calculate_dynamic_mu", "FlowMatchSchedulePolicy", "ensure_req_sigmas"]
