"""Adapter injection: LoRA, the dual-adapter NFT setup, and full-weight mirrors.

Native modules keep *fused* weights (``qkv_proj``, ``gate_up_proj``), so an adapter targets a row
block of a fused weight: a module advertises its blocks through ``lora_targets()`` →
``{hf_name: (param_name, row_offset, rows)}`` and calls :func:`lora_apply` after the base GEMM, which
adds ``scaling · (x·Aᵀ)·Bᵀ`` into that block.  State-dict keys follow the PEFT grammar
(``base_model.model.<path>.lora_A.<adapter>.weight``) so adapter checkpoints and the LoRA weight-sync
payloads interoperate with PEFT-based tooling.

``inject_nft`` creates two adapters — trainable ``default`` and frozen ``old`` — and returns a
:class:`AdapterShadow` whose ``use_shadow()`` routes forwards through ``old`` (DiffusionNFT's reference
policy) and whose EMA step pulls ``old`` toward ``default``.
Parity: ``unirl/train/inject.py:49-84`` (LoRA), ``:92-147`` (NFT), ``:155-181`` (mirror), ``:456-538`` (deferred ops).
"""

from __future__ import annotations

import contextlib
import math
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from unirl_b200.train.ema import ema_decay_at


class LoraAdapter(nn.Module):
    def __init__(self, in_features: int, rows: int, row_offset: int, rank: int, alpha: float, dropout: float, dtype: torch.dtype, device: Any):
        super().__init__()
        self.row_offset, self.rows, self.rank = int(row_offset), int(rows), int(rank)
        self.scaling = float(alpha) / float(rank)
        self.dropout = float(dropout)
        self.lora_A = nn.Parameter(torch.empty(rank, in_features, dtype=dtype, device=device))
        self.lora_B = nn.Parameter(torch.zeros(rows, rank, dtype=dtype, device=device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    def delta(self, x: torch.Tensor) -> torch.Tensor:
        if self.dropout > 0 and self.training:
            x = F.dropout(x, self.dropout)
        return F.linear(F.linear(x, self.lora_A.to(x.dtype)), self.lora_B.to(x.dtype)) * self.scaling


def _key(target: str, adapter: str) -> str:
    return f"{target.replace('.', ':')}__{adapter}"  # module names may not contain dots


def _split_key(key: str) -> Tuple[str, str]:
    target, adapter = key.rsplit("__", 1)
    return target.replace(":", "."), adapter


def lora_apply(module: nn.Module, param_name: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Add the active adapters' low-rank updates for ``param_name`` into ``y`` (no-op without adapters)."""
    table = getattr(module, "_lora_index", None)
    if not table or param_name not in table:
        return y
    active = getattr(module, "_lora_active", "default")
    parts = []  # (row_offset, rows, delta) of every active adapter on this fused weight
    for target in table[param_name]:
        ad = module.lora[_key(target, active)] if _key(target, active) in module.lora else None
        if ad is not None:
            parts.append((ad.row_offset, ad.rows, ad.delta(x)))
    if not parts:
        return y
    parts.sort(key=lambda p: p[0])
    width = y.shape[-1]
    if len(parts) == 1 and parts[0][0] == 0 and parts[0][1] == width:
        return y + parts[0][2]
    # Adapters on named row ranges of one fused weight (q | k | v, gate | up): assemble ONE full-width update and add it once,
    # instead of re-assembling the whole output per adapter.  Ranges without an adapter get zeros.
    cols, cursor = [], 0
    for off, rows, d in parts:
        if off < cursor:
            raise ValueError(f"overlapping adapters on {param_name}")
        if off > cursor:
            cols.append(d.new_zeros(*d.shape[:-1], off - cursor))
        cols.append(d)
        cursor = off + rows
    if cursor < width:
        cols.append(parts[0][2].new_zeros(*parts[0][2].shape[:-1], width - cursor))
    return y + torch.cat(cols, -1)


def _hosts(model: nn.Module) -> Iterator[Tuple[str, nn.Module]]:
    for name, mod in model.named_modules():
        if callable(getattr(mod, "lora_targets", None)):
            yield name, mod


def inject_lora(model: nn.Module, *, rank: int, alpha: float, target_modules: Sequence[str], dropout: float = 0.0,
                adapter_name: str = "default", trainable: bool = True, freeze_base: bool = True, **_ignored: Any) -> int:
    """Attach one adapter per matching target; returns the number of adapters created."""
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    made = 0
    want = set(target_modules)
    for _name, mod in _hosts(model):
        targets: Dict[str, Tuple[str, int, int]] = mod.lora_targets()
        if not hasattr(mod, "lora"):
            mod.lora = nn.ModuleDict()
            mod._lora_index = {}
            mod._lora_active = "default"
        for target, (param_name, off, rows) in targets.items():
            # a recipe's pattern may carry more of the module path than the target's name ("attn.to_q" for "to_q") or less ("gate_proj" for "mlp.gate_proj")
            if not any(w == target or w.endswith("." + target) or target.endswith("." + w) for w in want):
                continue
            w = getattr(mod, param_name)
            ad = LoraAdapter(w.shape[1], rows, off, rank, alpha, dropout, w.dtype, w.device)
            for p in ad.parameters():
                p.requires_grad_(trainable)
            mod.lora[_key(target, adapter_name)] = ad
            mod._lora_index.setdefault(param_name, [])
            if target not in mod._lora_index[param_name]:
                mod._lora_index[param_name].append(target)
            made += 1
    if made == 0:
        raise ValueError(f"inject_lora: no module exposes any of the targets {sorted(want)}")
    return made


class AdapterShadow:
    """EMA handle over a ``default`` / ``old`` adapter pair (the NFT "LoRA policy")."""

    def __init__(self, model: nn.Module, default: str, shadow: str):
        self.model, self.default, self.shadow = model, default, shadow
        self.decay, self.decay_type, self.timing, self.decay_kw = 0.001, "constant", "rollout_end", {}
        self.sharded = None

    def bind(self, sharded: Any) -> None:
        self.sharded = sharded
        self.copy_default_to_shadow()

    def configure(self, *, decay: float, decay_type: str, timing: str, flat_steps: int = 0, uprate: float = 0.001, uphold: float = 0.5) -> None:
        self.decay, self.decay_type, self.timing = float(decay), decay_type, timing
        self.decay_kw = dict(flat_steps=flat_steps, uprate=uprate, uphold=uphold)

    def iter_pairs(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for _n, mod in _hosts(self.model):
            if not hasattr(mod, "lora"):
                continue
            for key, ad in mod.lora.items():
                target, adapter = _split_key(key)
                if adapter == self.default and _key(target, self.shadow) in mod.lora:
                    sh = mod.lora[_key(target, self.shadow)]
                    yield ad.lora_A, sh.lora_A
                    yield ad.lora_B, sh.lora_B

    @torch.no_grad()
    def copy_default_to_shadow(self) -> None:
        for live, shd in self.iter_pairs():
            shd.copy_(live)

    @torch.no_grad()
    def _lerp(self, t: int) -> None:
        d = ema_decay_at(t, self.decay, self.decay_type, **self.decay_kw)
        for live, shd in self.iter_pairs():
            shd.mul_(d).add_(live.to(shd.dtype), alpha=1.0 - d)

    def step(self, t: int) -> None:
        if self.timing == "optimizer_step":
            self._lerp(t)

    def on_rollout_end(self, t: int) -> None:
        if self.timing == "rollout_end":
            self._lerp(t)

    def _set_active(self, adapter: str) -> None:
        for _n, mod in _hosts(self.model):
            if hasattr(mod, "lora"):
                mod._lora_active = adapter

    def apply_shadow(self) -> None:
        self._set_active(self.shadow)

    def restore_shadow(self) -> None:
        self._set_active(self.default)

    swap_in, swap_out = apply_shadow, restore_shadow

    @contextlib.contextmanager
    def use_shadow(self) -> Iterator[None]:
        self.apply_shadow()
        try:
            yield
        finally:
            self.restore_shadow()


Shadow = AdapterShadow


def inject_nft(model: nn.Module, *, rank: int, alpha: float, target_modules: Sequence[str], default: str = "default", shadow: str = "old",
               dropout: float = 0.0, **_ignored: Any) -> AdapterShadow:
    inject_lora(model, rank=rank, alpha=alpha, target_modules=target_modules, dropout=dropout, adapter_name=default, trainable=True)
    inject_lora(model, rank=rank, alpha=alpha, target_modules=target_modules, dropout=0.0, adapter_name=shadow, trainable=False, freeze_base=False)
    return AdapterShadow(model, default, shadow)


def inject_mirror(model: nn.Module, prefix: str = "shadow_") -> None:
    """Full-weight EMA is kept on the optimizer shards (``ShardEMA``); nothing to inject into the module."""
    return None


# ---- PEFT key grammar -------------------------------------------------------------------------------------
def lora_named_tensors(model: nn.Module, adapter: str = "default", prefix: str = "base_model.model.") -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name, mod in _hosts(model):
        if not hasattr(mod, "lora"):
            continue
        hf_path = getattr(mod, "hf_module_path", lambda t: f"{name}.{t}")
        for key, ad in mod.lora.items():
            target, ad_name = _split_key(key)
            if ad_name != adapter:
                continue
            base = f"{prefix}{hf_path(target)}"
            out[f"{base}.lora_A.{adapter}.weight"] = ad.lora_A
            out[f"{base}.lora_B.{adapter}.weight"] = ad.lora_B
    return out


def peft_config_dict(rank: int, alpha: float, target_modules: Sequence[str]) -> Dict[str, Any]:
    return {"peft_type": "LORA", "r": int(rank), "lora_alpha": float(alpha), "target_modules": list(target_modules), "lora_dropout": 0.0,
            "bias": "none", "task_type": "FEATURE_EXTRACTION"}


__all__ = ["LoraAdapter", "lora_apply", "inject_lora", "inject_nft", "inject_mirror", "AdapterShadow", "Shadow", "lora_named_tensors", "peft_config_dict"]
