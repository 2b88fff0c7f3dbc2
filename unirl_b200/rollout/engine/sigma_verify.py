"""σ-schedule echo check: an engine returns the schedule it actually ran; the trainer refuses to train on a mismatch.

Engines may report timesteps on a ``0…1000`` scale instead of ``0…1``; a reported maximum above 10 is taken as scaled
by ``round(max_reported / max_expected)`` and divided out before the comparison.  A difference beyond
``atol=1e-5, rtol=1e-4`` is fatal: replaying a trajectory under another schedule silently biases every log-prob.
Parity: ``unirl/rollout/engine/sigma_verify.py:67-139``.
"""

from __future__ import annotations

from typing import Any

import torch


class SigmaMismatchError(RuntimeError):
    pass


def normalize_reported_sigmas(reported: torch.Tensor, expected: torch.Tensor) -> torch.Tensor:
    r = reported.detach().float().flatten().cpu()
    e = expected.detach().float().flatten().cpu()
    if r.numel() and float(r.max()) > 10.0 and float(e.max()) > 0:
        scale = round(float(r.max()) / float(e.max()))
        if scale > 0:
            r = r / float(scale)
    return r


def verify_sigmas(reported: Any, expected: Any, *, atol: float = 1e-5, rtol: float = 1e-4, who: str = "engine") -> None:
    if reported is None or expected is None:
        raise SigmaMismatchError(f"{who}: missing σ schedule (reported={reported is not None}, expected={expected is not None})")
    e = torch.as_tensor(expected).detach().float().flatten().cpu()
    r = normalize_reported_sigmas(torch.as_tensor(reported), e)
    if r.numel() == e.numel() - 1 and float(e[-1]) == 0.0:  # engines that drop the terminal 0
        e = e[:-1]
    if r.shape != e.shape:
        raise SigmaMismatchError(f"{who}: σ schedule has {r.numel()} entries, the request pinned {e.numel()}")
    if not torch.allclose(r, e, atol=atol, rtol=rtol):
        worst = int((r - e).abs().argmax())
        raise SigmaMismatchError(f"{who}: σ[{worst}] = {float(r[worst]):.6f} but the request pinned {float(e[worst]):.6f}")


__all__ = ["verify_sigmas", "normalize_reported_sigmas", "SigmaMismatchError"]
