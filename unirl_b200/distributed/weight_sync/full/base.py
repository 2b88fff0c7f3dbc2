"""``FullWeightSync`` — walk the trainer's weights and hand them to a rollout engine.

Shared by every full-weight handler: the weight walk (raw base weights, or LoRA folded in fp32 —
``base + (B·A)·alpha/r`` — when ``lora_merged``), the optional ``wire_dtype`` cast, ordered single-``*``
``name_remap`` rules (``None`` drops a tensor), size-bounded bucketing and the ``weight_version``
counter.  The bf16 replica is resident on every trainer rank (see ``parallel/flat_shard.py``), so the
walk needs no per-parameter all-gather, unlike the reference (``unirl/utils/peft_merge.py:17-29``).
Parity: ``unirl/distributed/weight_sync/full/base.py:28-56`` (remap), ``:59-113``, ``:119-159``, ``:161-178``.
"""

from __future__ import annotations

import time
from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch

from unirl_b200.config.require import require
from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.utils.dtypes import parse_torch_dtype
from unirl_b200.utils.peft_merge import merged_state_dict, raw_state_dict


def _one_star(s: object) -> bool:
    return isinstance(s, str) and s.count("*") == 1


def validate_name_remap(rules: Optional[Dict[str, Optional[str]]]) -> Dict[str, Optional[str]]:
    rules = dict(rules or {})
    keys = list(rules)
    for i, (k, v) in enumerate(rules.items()):
        require(_one_star(k), f"name_remap key {k!r} needs exactly one '*'")
        require(v is None or _one_star(v), f"name_remap[{k!r}] must be null or contain one '*', got {v!r}")
        require(k != "*" or i == len(keys) - 1, f"name_remap '*' must come last; it shadows {keys[i + 1:]!r}")
    return rules


def apply_name_remap(name: str, rules: Dict[str, Optional[str]]) -> Optional[str]:
    for k, v in rules.items():
        pre, _, post = k.partition("*")
        if name.startswith(pre) and name.endswith(post) and len(name) >= len(pre) + len(post):
            if v is None:
                return None
            vpre, _, vpost = v.partition("*")
            return vpre + name[len(pre) : len(name) - len(post)] + vpost
    return name


class FullWeightSync(Remote):
    def __init__(self, *, backend: Any, rollout: Any = None, bucket_size_mb: int = 512, flush_cache: bool = True, lora_merged: bool = False,
                 name_remap: Optional[Dict[str, Optional[str]]] = None, track_prefix: str = "", wire_dtype: Any = None,
                 use_merged: Optional[bool] = None, param_name_prefix: Optional[str] = None, target_modules: Any = None) -> None:
        """The last three are earlier spellings that some recipes of the reference still carry (its
        ``examples/diffusion/hunyuan_video15_t2v_vllmomni_nccl_separate.yaml:214-221``): ``use_merged`` is ``lora_merged``,
        ``param_name_prefix`` is ``track_prefix``, and ``target_modules`` named the one module this class always sends."""
        super().__init__()
        lora_merged = bool(lora_merged) if use_merged is None else bool(use_merged)
        track_prefix = track_prefix or (param_name_prefix or "")
        self.target_modules = None if target_modules is None else list(target_modules)
        self._backend, self._rollout = backend, rollout
        self._bucket_bytes = int(bucket_size_mb) * 1024 * 1024
        self._flush_cache, self._lora_merged = bool(flush_cache), bool(lora_merged)
        self._name_remap = validate_name_remap(name_remap)
        self._track_prefix = str(track_prefix or "")
        self._wire_dtype = None if wire_dtype is None else parse_torch_dtype(wire_dtype)
        self.weight_version = 0
        self.last_sync_ms = 0.0

    def _iter_full_tensors(self) -> Iterator[Tuple[str, torch.Tensor]]:
        walk = merged_state_dict if self._lora_merged else raw_state_dict
        for name, t in walk(self._backend.model, dtype=self._wire_dtype):
            if not self._lora_merged and (".lora_A" in name or ".lora_B" in name):
                continue
            out = apply_name_remap(name, self._name_remap)
            if out is not None:
                yield out, t

    def _iter_buckets(self) -> Iterator[Tuple[List[Tuple[str, torch.Tensor]], bool]]:
        bucket: List[Tuple[str, torch.Tensor]] = []
        size = 0
        for name, t in self._iter_full_tensors():
            n = t.numel() * t.element_size()
            if bucket and size + n >= self._bucket_bytes:
                yield bucket, False
                bucket, size = [], 0
            bucket.append((name, t))
            size += n
        if bucket:
            yield bucket, True

    def _timed(self, fn) -> Any:
        """Device-timed section (CUDA events) → ``last_sync_ms``."""
        if torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            b.synchronize()
            self.last_sync_ms = a.elapsed_time(b)
            return out
        t0 = time.perf_counter()
        out = fn()
        self.last_sync_ms = (time.perf_counter() - t0) * 1e3
        return out

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sync(self) -> Dict[str, float]:
        raise NotImplementedError

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def get_weight_version(self) -> int:
        return self.weight_version


__all__ = ["FullWeightSync", "validate_name_remap", "apply_name_remap"]
