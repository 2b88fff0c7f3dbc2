"""Deterministic initial noise: per-group seeds from a hash, draws pinned to CPU fp32.

``seed(group) = blake2b_8("{base_seed}::{group_id}") mod 2^63`` so shards that see the same
``(base_seed, group ids)`` reproduce the same x_T regardless of how the batch was split; the draw
always happens on CPU in fp32 (bit-stable across machines, unlike device RNGs) and only then is
moved / cast.  Parity: ``unirl/sde/noise.py:26-95``, ``:98-152``, ``:155-187``.
"""

from __future__ import annotations

import hashlib
from typing import Dict, List, Optional, Sequence, Tuple

import torch

MAX_TORCH_SEED = (1 << 63) - 1


def derive_group_seed(base_seed: int, group_id: str) -> int:
    digest = hashlib.blake2b(f"{int(base_seed)}::{group_id}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "big") % (MAX_TORCH_SEED + 1)


_derive_group_seed = derive_group_seed


def generate_shared_noise(batch_size: int, latent_shape: Tuple[int, ...], device, dtype: torch.dtype = torch.float32,
                          noise_group_ids: Optional[List[str]] = None, base_seed: Optional[int] = None) -> torch.Tensor:
    """``[B, *latent_shape]`` noise where equal group ids share one draw."""
    if not isinstance(noise_group_ids, list) or len(noise_group_ids) != batch_size:
        raise ValueError(f"generate_shared_noise needs one noise_group_id per sample (batch {batch_size}, got "
                         f"{len(noise_group_ids) if isinstance(noise_group_ids, list) else None})")
    cache: Dict[str, torch.Tensor] = {}
    rows = []
    for gid in map(str, noise_group_ids):
        if gid not in cache:
            gen = None
            if base_seed is not None:
                gen = torch.Generator(device=device)
                gen.manual_seed(derive_group_seed(base_seed, gid))
            cache[gid] = torch.randn(*latent_shape, device=device, dtype=dtype, generator=gen)
        rows.append(cache[gid])
    return torch.stack(rows)


def generate_latents(batch_size: int, latent_shape: Tuple[int, ...], device, dtype: torch.dtype = torch.float32,
                     init_same_noise: bool = False, samples_per_prompt: int = 1, noise_group_ids: Optional[List[str]] = None,
                     base_seed: Optional[int] = None) -> torch.Tensor:
    if init_same_noise:
        if base_seed is None or noise_group_ids is None:
            raise ValueError("init_same_noise=True needs base_seed and noise_group_ids")
        return generate_shared_noise(batch_size, latent_shape, device, dtype, noise_group_ids, base_seed)
    return torch.randn(batch_size, *latent_shape, device=device, dtype=dtype)


def regen_initial_noise(noise_group_ids: Sequence[str], base_seed: int, latent_shape: Tuple[int, ...], device,
                        dtype: torch.dtype = torch.float32) -> torch.Tensor:
    x = generate_shared_noise(len(noise_group_ids), tuple(latent_shape), torch.device("cpu"), torch.float32,
                              list(noise_group_ids), int(base_seed))
    return x.to(device=device, dtype=dtype)


def step_noise_seed(base_seed: int, group_id: str, step: int) -> int:
    """Seed for the per-step SDE noise of one sample (keeps rollout and replay aligned per sample)."""
    return derive_group_seed(base_seed, f"{group_id}@step{int(step)}")


__all__ = ["MAX_TORCH_SEED", "derive_group_seed", "generate_shared_noise", "generate_latents", "regen_initial_noise", "step_noise_seed"]
