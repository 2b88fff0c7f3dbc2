"""State-dict helpers for the sharded backend.

The bf16 replica is resident on every rank, so a "full state dict" is a local read (the
reference needs a DCP gather, ``unirl/train/fsdp_utils.py:15-88``); models that define
``hf_state_dict`` / ``load_hf_state_dict`` are saved in the Hugging Face key grammar so the
``policy_state_dict`` in ``checkpoint.pt`` stays interchangeable.  A per-tensor SHA-256/16 manifest
is written beside the checkpoint for integrity checks.
"""

from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Iterator, Tuple

import torch
import torch.nn as nn


def full_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    if hasattr(model, "hf_state_dict"):
        return dict(model.hf_state_dict())
    return dict(model.state_dict())


@torch.no_grad()
def load_full_state_dict(model: nn.Module, sd: Dict[str, torch.Tensor], strict: bool = True) -> None:
    if hasattr(model, "load_hf_state_dict") and strict:
        model.load_hf_state_dict(sd)
        return
    own = full_state_dict(model)
    missing = [k for k in own if k not in sd]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"state dict mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    for k, v in sd.items():
        if k in own:
            own[k].copy_(v.to(own[k]))


def trainable_params(model: nn.Module) -> Iterator[nn.Parameter]:
    return (p for p in model.parameters() if p.requires_grad)


def lora_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v for k, v in full_state_dict(model).items() if "lora_A" in k or "lora_B" in k}


def nft_state_dict(model: nn.Module, adapter: str = "default") -> Dict[str, torch.Tensor]:
    return {k: v for k, v in lora_state_dict(model).items() if f".{adapter}." in k}


def clip_grad_norm(params: Iterable[nn.Parameter], max_norm: float, comm=None) -> torch.Tensor:
    """Explicit sharded clip: local Σg² → all-reduce(SUM) → scale.  (Used for modules outside the flat runtime.)"""
    params = [p for p in params if p.grad is not None]
    total = torch.stack([p.grad.float().pow(2).sum() for p in params]).sum() if params else torch.zeros(())
    if comm is not None:
        total = comm.all_reduce(total.reshape(1)).reshape(())
    norm = total.sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad))
    return norm


def write_manifest(path: str, sd: Dict[str, torch.Tensor]) -> None:
    from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor

    with open(os.path.join(path, "manifest.json"), "w") as f:
        json.dump({k: fingerprint_tensor(v) for k, v in sd.items()}, f)


def verify_manifest(path: str, sd: Dict[str, torch.Tensor]) -> Tuple[bool, list]:
    from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor

    with open(os.path.join(path, "manifest.json")) as f:
        want = json.load(f)
    bad = [k for k, v in sd.items() if want.get(k) != fingerprint_tensor(v)]
    return not bad, bad


__all__ = ["full_state_dict", "load_full_state_dict", "trainable_params", "lora_state_dict", "nft_state_dict", "clip_grad_norm",
           "write_manifest", "verify_manifest"]
