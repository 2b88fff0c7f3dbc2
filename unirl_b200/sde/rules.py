"""Naming rules for SDE types.  Parity: ``unirl/sde/rules.py``."""

from __future__ import annotations

from typing import Any

_ALIASES = {"flow": "sde", "flow_sde": "sde", "sde": "sde", "cps": "cps", "dance": "dance", "dancegrpo": "dance",
            "ode": "ode", "dpm2": "dpm2", "dpm": "dpm2"}


def normalize_sde_type(value: Any) -> str:
    key = str(getattr(value, "canonical_name", value)).strip().lower()
    if key not in _ALIASES:
        raise ValueError(f"unknown sde type {value!r}")
    return _ALIASES[key]


def is_deterministic_sde_type(value: Any, eta: float = 1.0) -> bool:
    return normalize_sde_type(value) in ("ode", "dpm2") or float(eta) < 1e-7


__all__ = ["normalize_sde_type", "is_deterministic_sde_type"]
