"""Temporarily run a model on another of its LoRA adapters.

Adapters here live on the host modules of ``train/inject.py`` (``mod.lora`` keyed by target and adapter name, ``mod._lora_active`` naming
the adapter the forward pass applies).  The flat-sharded trainer keeps the module tree intact, so the same walk serves wrapped and
unwrapped models.  Parity: ``unirl/utils/adapter_utils.py`` (``switch_adapter``).
"""

from __future__ import annotations

import contextlib
from typing import Iterator, List, Tuple

import torch.nn as nn


def adapter_hosts(model: nn.Module) -> List[nn.Module]:
    model = getattr(model, "module", model)
    return [m for m in model.modules() if hasattr(m, "lora")]


def adapter_names(model: nn.Module) -> List[str]:
    from unirl_b200.train.inject import _split_key

    return sorted({_split_key(k)[1] for m in adapter_hosts(model) for k in m.lora})


@contextlib.contextmanager
def switch_adapter(model: nn.Module, adapter_name: str) -> Iterator[None]:
    """Inside the block every adapter host applies ``adapter_name``; the adapter each host was using before comes back afterwards,
    also when the block raises.  A model without adapters passes through unchanged; an unknown name is an error."""
    hosts = adapter_hosts(model)
    if hosts and adapter_name not in adapter_names(model):
        raise KeyError(f"no adapter named {adapter_name!r}; the model carries {adapter_names(model)}")
    before: List[Tuple[nn.Module, str]] = [(m, getattr(m, "_lora_active", "default")) for m in hosts]
    try:
        for m in hosts:
            m._lora_active = adapter_name
        yield
    finally:
        for m, name in before:
            m._lora_active = name


__all__ = ["switch_adapter", "adapter_names", "adapter_hosts"]
