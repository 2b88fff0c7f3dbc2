"""Weight walks for sync / export: raw base weights, LoRA-merged weights, LoRA tensor extraction, engine adapters.

``merged_state_dict`` folds every adapter into its base block in fp32 — ``W[rows] += (B·A)·alpha/r`` — and
yields the module's native (fused) names; ``extract_lora_tensors`` yields canonical PEFT-style names
``<prefix><module>.lora_{A,B}.weight`` with a dtype guard.  Parity: ``unirl/utils/peft_merge.py:17-29``
(full-tensor materialisation — a local read here), ``:32-109`` (merged walk), ``:112-159`` (raw walk),
``:162-207`` (LoRA extraction), ``:210-276`` (engine adapters).
"""

from __future__ import annotations

from typing import Any, Dict, Iterator, Optional, Tuple

import torch
import torch.nn as nn


def _key(target: str, adapter: str) -> str:
    from unirl_b200.train.inject import _key as k

    return k(target, adapter)


def _cast(t: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    return t.to(dtype) if dtype is not None and t.is_floating_point() and t.dtype != dtype else t


def raw_state_dict(model: nn.Module, dtype: Optional[torch.dtype] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, p in model.named_parameters():
        yield name, (p.detach() if ".lora." in name else _cast(p.detach(), dtype))


def merged_state_dict(model: nn.Module, dtype: Optional[torch.dtype] = None, adapter: str = "default") -> Iterator[Tuple[str, torch.Tensor]]:
    hosts = {n: m for n, m in model.named_modules() if getattr(m, "_lora_index", None)}
    for name, p in model.named_parameters():
        if ".lora." in name:
            continue
        owner, _, leaf = name.rpartition(".")
        host = hosts.get(owner)
        if host is None or leaf not in host._lora_index:
            yield name, _cast(p.detach(), dtype)
            continue
        w = p.detach().float().clone()
        for target in host._lora_index[leaf]:
            key = _key(target, adapter)
            if key in host.lora:
                ad = host.lora[key]
                w[ad.row_offset : ad.row_offset + ad.rows] += (ad.lora_B.detach().float() @ ad.lora_A.detach().float()) * ad.scaling
        yield name, w.to(dtype or p.dtype)


def extract_lora_tensors(model: nn.Module, adapter: str = "default", prefix: str = "") -> Dict[str, torch.Tensor]:
    from unirl_b200.train.inject import lora_named_tensors

    out = {}
    for k, v in lora_named_tensors(model, adapter, prefix="").items():
        if v.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise TypeError(f"LoRA tensor {k} has unsupported dtype {v.dtype}")
        canon = k.replace(f".lora_A.{adapter}.weight", ".lora_A.weight").replace(f".lora_B.{adapter}.weight", ".lora_B.weight")
        out[prefix + canon] = v.detach().cpu()
    return out


def adapt_lora_for_engine(tensors: Dict[str, torch.Tensor], *, strip_prefix: str = "", add_prefix: str = "", alpha: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """Rename for a receiving engine: strip the pipeline prefix, add the engine's, optionally inject per-module ``.alpha`` scalars."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in tensors.items():
        name = k[len(strip_prefix):] if strip_prefix and k.startswith(strip_prefix) else k
        out[add_prefix + name] = v
        if alpha is not None and name.endswith(".lora_A.weight"):
            out[add_prefix + name[: -len(".lora_A.weight")] + ".alpha"] = torch.tensor(float(alpha))
    return out


def adapt_lora_for_vllm(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return adapt_lora_for_engine(tensors, add_prefix="base_model.model.")


def adapt_lora_for_sglang(tensors: Dict[str, torch.Tensor], pipeline_prefix: str = "transformer.", alpha: Optional[float] = None) -> Dict[str, torch.Tensor]:
    return adapt_lora_for_engine(tensors, strip_prefix=pipeline_prefix, alpha=alpha)


__all__ = ["raw_state_dict", "merged_state_dict", "extract_lora_tensors", "adapt_lora_for_engine", "adapt_lora_for_vllm", "adapt_lora_for_sglang"]
