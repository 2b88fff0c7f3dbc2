"""Contracts every model package implements.

``Bundle``   – pure container of modules (trainable transformer + frozen aux) and a tokenizer.
``Pipeline`` – ``generate(RolloutReq) -> RolloutResp`` for one bundle, composed of stages.
``ARStage``  – ``autoregress(conditions, sampling_params) -> TextSegment``; ``replay(conditions, segment, temperature)``
               → packed ``[total_tokens]`` log-probs (differentiable).
``DiffusionStage`` – ``diffuse`` / ``replay`` / ``predict_noise_at_step``.
``ReplayResult``   – ``(log_probs [B,S'], prev_sample_means [B,S',…], logits)``.

Parity: ``unirl/models/types/{bundle,pipeline,ar,diffusion,codec,embedding,replay_result}.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Generic, List, Optional, Protocol, Tuple, TypeVar, runtime_checkable

import torch

from unirl_b200.distributed.group.remote import Remote

C = TypeVar("C")
P = TypeVar("P")


class Bundle(Remote):
    """Collection of related modules that a pipeline's stages dispatch against."""

    def trainable_modules(self) -> dict:
        return {"transformer": getattr(self, "transformer")}

    def materialize(self, device: Any, with_aux: bool = True) -> None:
        """Move / allocate weights on ``device`` (meta-initialised bundles fill their shards here)."""
        for m in self.trainable_modules().values():
            m.to(device)


class Pipeline(Remote):
    def generate(self, req: Any) -> Any:
        raise NotImplementedError


class LatentShapeProvider(Protocol):
    @classmethod
    def latent_shape(cls, *, model_config: Any, sampling_spec: Any) -> Tuple[int, ...]: ...


@dataclass
class ReplayResult:
    log_probs: Optional[torch.Tensor] = None
    prev_sample_means: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None


@runtime_checkable
class ARStage(Protocol[C]):
    def autoregress(self, conditions: C, *, sampling_params: Any, **kw: Any) -> Any: ...

    def replay(self, conditions: C, *, segment: Any, temperature: float = 1.0) -> torch.Tensor: ...


@runtime_checkable
class ARStep(Protocol):
    def step(self, logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]: ...


@runtime_checkable
class DiffusionStep(Protocol):
    def forward(self, *, strategy: Any, noise_pred: torch.Tensor, sample: torch.Tensor, sigma: torch.Tensor, sigma_next: torch.Tensor,
                prev_sample: Optional[torch.Tensor] = None, sigma_max: float = 0.99, eta: float = 1.0, step_index: int = 0): ...


@runtime_checkable
class DiffusionStage(Protocol[C]):
    def diffuse(self, conditions: C, *, schedule: torch.Tensor, params: Any) -> Any: ...

    def replay(self, conditions: C, *, segment: Any, params: Any, step_indices: Optional[List[int]] = None) -> ReplayResult: ...

    def predict_noise_at_step(self, conditions: C, *, sample: torch.Tensor, sigma: torch.Tensor, params: Any) -> torch.Tensor: ...


@runtime_checkable
class EmbedStage(Protocol[P, C]):
    def embed(self, p: P) -> C: ...


@runtime_checkable
class EncodeStage(Protocol[P]):
    def encode(self, p: P) -> torch.Tensor: ...


@runtime_checkable
class DecodeStage(Protocol[P]):
    def decode(self, latents: torch.Tensor) -> P: ...


def left_pad_prompt(input_ids: torch.Tensor, attention_mask: torch.Tensor, pad_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Right-padded ``[real | pad]`` rows → left-padded ``[pad | real]`` trimmed to the longest real length."""
    lens = attention_mask.long().sum(1)
    if not lens.numel() or int(lens.max()) == 0:
        return input_ids, attention_mask
    width = int(lens.max())
    ids = torch.full((input_ids.shape[0], width), int(pad_id), dtype=input_ids.dtype, device=input_ids.device)
    mask = torch.zeros((input_ids.shape[0], width), dtype=attention_mask.dtype, device=input_ids.device)
    keep = attention_mask.bool()
    for b, n in enumerate(lens.tolist()):
        if n:
            ids[b, width - n :] = input_ids[b][keep[b]][:width]
            mask[b, width - n :] = 1
    return ids, mask


def unpad_prompts(input_ids: torch.Tensor, attention_mask: torch.Tensor) -> List[torch.Tensor]:
    """Per-row real tokens of a padded prompt batch (either padding side)."""
    keep = attention_mask.bool()
    return [input_ids[b][keep[b]] for b in range(input_ids.shape[0])]


__all__ = ["Bundle", "Pipeline", "LatentShapeProvider", "ReplayResult", "ARStage", "ARStep", "DiffusionStep", "DiffusionStage",
           "EmbedStage", "EncodeStage", "DecodeStage", "left_pad_prompt", "unpad_prompts"]
