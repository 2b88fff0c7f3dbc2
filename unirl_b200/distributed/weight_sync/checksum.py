"""Tensor fingerprints used to prove weight-sync / checkpoint parity.

``fingerprint_tensor`` = first 16 hex chars of SHA-256 over ``dtype | shape | raw bytes`` — the
reference's criterion (``unirl/rollout/engine/vllm_omni/weight_sync/checksum.py:32-55``).  LoRA
checksums are order-free multisets with ``lora_B`` pre-scaled by ``alpha / r`` so engines that fold
the scaling into B compare equal (``:58-108``).
"""

from __future__ import annotations

import hashlib
from collections import Counter
from typing import Dict, Iterable, Mapping, Tuple

import torch


def fingerprint_tensor(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    h = hashlib.sha256()
    h.update(str(t.dtype).encode())
    h.update(str(tuple(t.shape)).encode())
    h.update(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    return h.hexdigest()[:16]


def fingerprint_named(tensors: Mapping[str, torch.Tensor]) -> Dict[str, str]:
    return {k: fingerprint_tensor(v) for k, v in tensors.items()}


def lora_checksum_multiset(tensors: Mapping[str, torch.Tensor], alpha: float, rank: int) -> Counter:
    scale = float(alpha) / float(rank)
    out: Counter = Counter()
    for name, t in tensors.items():
        out[fingerprint_tensor((t.float() * scale).to(t.dtype) if "lora_B" in name else t)] += 1
    return out


def compare_checksums(a: Mapping[str, str], b: Mapping[str, str]) -> Tuple[bool, list]:
    bad = sorted(k for k in set(a) | set(b) if a.get(k) != b.get(k))
    return not bad, bad


__all__ = ["fingerprint_tensor", "fingerprint_named", "lora_checksum_multiset", "compare_checksums"]
