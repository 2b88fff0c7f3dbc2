"""``RewardService`` — worker-side scoring of a rollout track.

``score_and_attach(req, track)`` (``DP_SCATTER``) builds a ``RewardRequest`` from the request's primitives
(replicated N×M for composed prompt-enhancement tracks) and the track's decoded output (plus raw
response tokens for token-level rule rewards), fails fast on any per-sample failure flag, applies AR
truncation shaping — ``zero`` | ``keep`` | ``soft`` (graded over-length penalty over the last
``overlong_buffer_len`` tokens) — and returns a copy of the track with ``rewards`` /
``component_rewards`` attached.  Parity: ``unirl/reward/service.py:111-140``, ``:155-275``, ``:277-287``.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.reward.base import RewardBackend
from unirl_b200.types.reward import RewardRequest, RewardResponse
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutTrack
from unirl_b200.types.sampling import get_ar_params, get_diffusion_params

logger = logging.getLogger(__name__)


def _generated_of(track: RolloutTrack, kind: str) -> Dict[str, Any]:
    gen: Dict[str, Any] = {}
    if track.decoded is not None:
        gen[kind] = track.decoded
    seg = track.segment
    if seg is not None and getattr(seg, "tokens", None) is not None and seg.cu_seqlens is not None:
        cu = seg.cu_seqlens.tolist()
        gen["tokens"] = [seg.tokens[cu[i] : cu[i + 1]] for i in range(len(cu) - 1)]
    if seg is not None and getattr(seg, "latents", None) is not None:
        gen["latents"] = seg.latents[:, -1]
    return gen


class RewardService(Remote):
    def __init__(self, backend: RewardBackend, truncated_reward: str = "zero", overlong_buffer_len: int = 4096,
                 overlong_penalty_factor: float = 1.0) -> None:
        super().__init__()
        self.backend = backend
        self.truncated_reward = str(truncated_reward)
        self.overlong_buffer_len, self.overlong_penalty_factor = int(overlong_buffer_len), float(overlong_penalty_factor)
        if self.truncated_reward not in ("zero", "keep", "soft"):
            raise ValueError(f"truncated_reward must be zero|keep|soft, got {self.truncated_reward!r}")

    @property
    def preferred_input_kind(self) -> str:
        kind = str(getattr(self.backend, "preferred_input_kind", "") or "").lower()
        if kind not in ("image", "video", "text"):
            raise ValueError(f"reward backend must expose preferred_input_kind image|video|text, got {kind!r}")
        return kind

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        return self.backend.compute_rewards(request)

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def score_and_attach(self, *, req: RolloutReq, track: RolloutTrack) -> RolloutTrack:
        if track.rewards is not None:
            raise RuntimeError("score_and_attach: the track already carries rewards")
        ids = list(track.sample_ids)
        prims = dict(req.primitives)
        metadata = list(req.metadata) if req.metadata else None
        req_n = next((len(v) for v in prims.values() if v is not None), 0)
        if req_n and req_n != len(ids):
            if len(ids) % req_n:
                raise RuntimeError(f"score_and_attach: request batch {req_n} does not divide track batch {len(ids)}")
            factor = len(ids) // req_n
            ar, df = get_ar_params(req.sampling_params), get_diffusion_params(req.sampling_params)
            n = int(ar.samples_per_prompt) if ar is not None else 1
            m = int(df.samples_per_prompt) if df is not None and hasattr(req.sampling_params, "diffusion") else 1
            if factor != n * m:
                raise RuntimeError(f"score_and_attach: expansion factor {factor} does not match sampling N*M = {n}*{m}")
            prims = {k: v.repeat_interleave(factor) for k, v in prims.items()}
            metadata = [x for x in metadata for _ in range(factor)] if metadata else None
        request = RewardRequest(primitives=prims, generated=_generated_of(track, self.preferred_input_kind),
                                metadata=metadata if metadata and any(x is not None for x in metadata) else None,
                                prompt_ids=[str(s) for s in ids], sample_ids=ids, group_ids=list(track.group_ids))
        resp = self.compute_rewards(request)
        failed = [(i, e) for i, (ok, e) in enumerate(zip(resp.successes, resp.errors)) if not ok]
        if failed:
            raise RuntimeError(f"reward computation failed for {len(failed)} of {len(resp.successes)} samples, e.g. {failed[:3]}")
        rewards = torch.tensor(resp.rewards, dtype=torch.float32)
        ar = get_ar_params(req.sampling_params)
        lens = getattr(track.segment, "lengths", None) if track.segment is not None else None
        if self.truncated_reward != "keep" and ar is not None and lens is not None and lens.numel() == rewards.numel():
            lens_f, max_len = lens.float().cpu(), float(int(ar.max_new_tokens))
            if self.truncated_reward == "zero":
                rewards = torch.where(lens_f >= max_len, torch.zeros_like(rewards), rewards)
            else:
                buf = float(self.overlong_buffer_len)
                rewards = rewards + torch.clamp(-(lens_f - (max_len - buf)) / buf * self.overlong_penalty_factor, max=0.0)
        comps = {str(k): torch.tensor(list(v or []), dtype=torch.float32) for k, v in dict(resp.component_rewards or {}).items()}
        return track.replace(rewards=rewards, component_rewards=comps)

    def is_available(self) -> bool:
        return self.backend.is_available()

    def offload(self) -> None:
        self.backend.offload()

    def onload(self) -> None:
        self.backend.onload()

    def dispose(self) -> None:
        self.backend.dispose()


__all__ = ["RewardService"]
