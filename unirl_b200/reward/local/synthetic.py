"""Token-level rule rewards for random-weight runs (no tokenizer, no dataset):

* ``LastTokenEvenReward``   – 1.0 if the last generated token id is even;
* ``TokenHashReward``       – 1.0 if a hash of the final ``window`` token ids ≡ 0 (mod ``modulus``);
* ``OptionLetterReward``    – 1.0 if the last emitted option-letter token equals a seeded target letter;
* ``LatentCNNReward`` / ``VideoConvReward`` – random-init conv scorers on final latents → scalar in [0, 1].
"""

from __future__ import annotations

import hashlib
import time
from typing import Any, List, Optional, Sequence

import torch
import torch.nn as nn

from unirl_b200.reward.base import RewardBackend
from unirl_b200.types.reward import RewardRequest, RewardResponse


class _TokenRule(RewardBackend):
    preferred_input_kind = "text"

    def score_tokens(self, toks: torch.Tensor, index: int, request: RewardRequest) -> float:
        raise NotImplementedError

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        toks = request.generated.get("tokens")
        if toks is None:
            raise ValueError(f"{type(self).__name__} needs generated['tokens']")
        r = [float(self.score_tokens(t, i, request)) for i, t in enumerate(toks)]
        return RewardResponse.ok(r, compute_time=time.perf_counter() - t0)


class LastTokenEvenReward(_TokenRule):
    def __init__(self, **_kw: Any):
        pass

    def score_tokens(self, toks, index, request):
        return 1.0 if toks.numel() and int(toks[-1]) % 2 == 0 else 0.0


class TokenHashReward(_TokenRule):
    def __init__(self, window: int = 16, modulus: int = 4, **_kw: Any):
        self.window, self.modulus = int(window), int(modulus)

    def score_tokens(self, toks, index, request):
        tail = toks[-self.window :].to(torch.int64).cpu().numpy().tobytes()
        return 1.0 if int.from_bytes(hashlib.blake2b(tail, digest_size=8).digest(), "big") % self.modulus == 0 else 0.0


class OptionLetterReward(_TokenRule):
    def __init__(self, option_token_ids: Sequence[int] = (32, 33, 34, 35, 36), seed: int = 0, **_kw: Any):
        self.options, self.seed = [int(x) for x in option_token_ids], int(seed)

    def target(self, sample_id: str) -> int:
        h = int.from_bytes(hashlib.blake2b(f"{self.seed}::{sample_id.split('/')[0]}".encode(), digest_size=8).digest(), "big")
        return self.options[h % len(self.options)]

    def score_tokens(self, toks, index, request):
        opts = torch.tensor(self.options)
        hit = torch.isin(toks.cpu(), opts).nonzero().flatten()
        if not hit.numel():
            return 0.0
        gid = (request.group_ids or request.sample_ids)[index]
        return 1.0 if int(toks[int(hit[-1])]) == self.target(str(gid)) else 0.0


class LatentCNNReward(RewardBackend):
    """Random-init 4-layer CNN on the final latent ``[B, C, H, W]`` → sigmoid scalar."""

    preferred_input_kind = "image"

    def __init__(self, in_channels: int = 16, width: int = 64, seed: int = 0, device: Optional[str] = None, **_kw: Any):
        g = torch.Generator().manual_seed(seed)
        chans = [in_channels, width, width * 2, width * 2, width * 4]
        layers: List[nn.Module] = []
        for a, b in zip(chans[:-1], chans[1:]):
            layers += [nn.Conv2d(a, b, 3, stride=2, padding=1), nn.SiLU()]
        self.net = nn.Sequential(*layers, nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(chans[-1], 1))
        with torch.no_grad():
            for p in self.net.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 / max(1.0, p.numel() ** 0.25)))
        self.device = device

    @torch.no_grad()
    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        x = request.generated.get("latents")
        if x is None:
            img = request.generated.get("image")
            x = getattr(img, "pixels", None)
        if x is None:
            raise ValueError("LatentCNNReward needs generated['latents'] or generated['image']")
        dev = torch.device(self.device) if self.device else x.device
        self.net.to(dev)
        if x.shape[1] != self.net[0].in_channels:
            x = x[:, : self.net[0].in_channels] if x.shape[1] > self.net[0].in_channels else torch.cat(
                [x, x.new_zeros(x.shape[0], self.net[0].in_channels - x.shape[1], *x.shape[2:])], 1)
        r = torch.sigmoid(self.net(x.to(dev).float())).flatten().cpu().tolist()
        return RewardResponse.ok(r, compute_time=time.perf_counter() - t0)


class VideoConvReward(RewardBackend):
    """Random-init 3-D conv scorer on the final video latent ``[B, C, F, H, W]`` → sigmoid scalar."""

    preferred_input_kind = "video"

    def __init__(self, in_channels: int = 16, width: int = 32, seed: int = 0, device: Optional[str] = None, **_kw: Any):
        g = torch.Generator().manual_seed(seed)
        self.net = nn.Sequential(nn.Conv3d(in_channels, width, 3, stride=(1, 2, 2), padding=1), nn.SiLU(),
                                 nn.Conv3d(width, width * 2, 3, stride=2, padding=1), nn.SiLU(),
                                 nn.Conv3d(width * 2, width * 4, 3, stride=2, padding=1), nn.SiLU(),
                                 nn.AdaptiveAvgPool3d(1), nn.Flatten(), nn.Linear(width * 4, 1))
        with torch.no_grad():
            for p in self.net.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 / max(1.0, p.numel() ** 0.25)))
        self.device = device

    @torch.no_grad()
    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        x = request.generated.get("latents")
        if x is None:
            raise ValueError("VideoConvReward needs generated['latents']")
        dev = torch.device(self.device) if self.device else x.device
        self.net.to(dev)
        r = torch.sigmoid(self.net(x.to(dev).float())).flatten().cpu().tolist()
        return RewardResponse.ok(r, compute_time=time.perf_counter() - t0)


__all__ = ["LastTokenEvenReward", "TokenHashReward", "OptionLetterReward", "LatentCNNReward", "VideoConvReward"]
