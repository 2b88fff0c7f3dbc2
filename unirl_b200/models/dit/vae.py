"""Latent codec (VAE) for image and video latents: native convolutional encoder / decoder.

Layout follows the KL auto-encoders the DiT families ship with: ``latent_channels`` at 1/8 resolution (1/4 in time for
video), residual blocks with group norm + SiLU, nearest-neighbour upsampling followed by a 3x3 convolution.  Decoding
runs in fp32 (``unirl/models/sd3/vae.py:34-56`` decodes in fp32 to avoid bf16 banding), ``scaling_factor`` /
``shift_factor`` map between model latents and codec latents.  Video latents ``[B, C, F, H, W]`` are decoded frame by
frame after a temporal expansion of ``temporal_factor`` (first frame kept single, as in causal video VAEs).

The codec is a frozen aux module: random-init unless a state dict in this module's key grammar is loaded.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VAEConfig:
    latent_channels: int = 16
    base_channels: int = 128
    channel_mult: Tuple[int, ...] = (1, 2, 4, 4)
    layers_per_block: int = 2
    scaling_factor: float = 1.5305
    shift_factor: float = 0.0609
    temporal_factor: int = 4
    groups: int = 32

    @classmethod
    def tiny(cls, latent_channels: int = 4) -> "VAEConfig":
        return cls(latent_channels, 8, (1, 1, 2, 2), 1, 1.0, 0.0, 4, 4)

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.channel_mult) - 1)


class _Res(nn.Module):
    def __init__(self, i: int, o: int, groups: int):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(min(groups, i), i), nn.Conv2d(i, o, 3, padding=1)
        self.n2, self.c2 = nn.GroupNorm(min(groups, o), o), nn.Conv2d(o, o, 3, padding=1)
        self.skip = nn.Conv2d(i, o, 1) if i != o else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.c1(F.silu(self.n1(x)))
        h = self.c2(F.silu(self.n2(h)))
        return h + (x if self.skip is None else self.skip(x))


class LatentVAE(nn.Module):
    def __init__(self, cfg: VAEConfig, device: Any = "cpu"):
        super().__init__()
        self.cfg = cfg
        ch = [cfg.base_channels * m for m in cfg.channel_mult]
        # decoder: deepest width first
        self.dec_in = nn.Conv2d(cfg.latent_channels, ch[-1], 3, padding=1)
        dec = []
        cur = ch[-1]
        for level in reversed(range(len(ch))):
            for _ in range(cfg.layers_per_block):
                dec.append(_Res(cur, ch[level], cfg.groups))
                cur = ch[level]
            if level > 0:
                dec.append(nn.Upsample(scale_factor=2.0, mode="nearest"))
                dec.append(nn.Conv2d(cur, cur, 3, padding=1))
        self.dec = nn.Sequential(*dec)
        self.dec_norm, self.dec_out = nn.GroupNorm(min(cfg.groups, cur), cur), nn.Conv2d(cur, 3, 3, padding=1)
        # encoder
        self.enc_in = nn.Conv2d(3, ch[0], 3, padding=1)
        enc = []
        cur = ch[0]
        for level in range(len(ch)):
            for _ in range(cfg.layers_per_block):
                enc.append(_Res(cur, ch[level], cfg.groups))
                cur = ch[level]
            if level < len(ch) - 1:
                enc.append(nn.Conv2d(cur, cur, 3, stride=2, padding=1))
        self.enc = nn.Sequential(*enc)
        self.enc_norm, self.enc_out = nn.GroupNorm(min(cfg.groups, cur), cur), nn.Conv2d(cur, 2 * cfg.latent_channels, 3, padding=1)
        self.to(device)

    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> "LatentVAE":
        g = torch.Generator(device="cpu").manual_seed(seed)
        for p in self.parameters():
            if p.dim() >= 2:
                fan_in = p[0].numel()
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, (1.0 / fan_in) ** 0.5, generator=g).to(p.device))
        return self.requires_grad_(False).eval()

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """Model latents → pixels in ``[0, 1]``; ``[B, C, H, W] → [B, 3, 8H, 8W]`` or ``[B, C, F, H, W] → [B, F', 3, 8H, 8W]``."""
        c = self.cfg
        z = latents.float() / c.scaling_factor + c.shift_factor
        video = z.dim() == 5
        if video:
            b, ch, f, h, w = z.shape
            reps = torch.tensor([1] + [c.temporal_factor] * (f - 1), device=z.device)
            z = z.repeat_interleave(reps, dim=2).permute(0, 2, 1, 3, 4).reshape(-1, ch, h, w)
        p = next(self.parameters())
        # The widest decoder activation is [n, 128, 8H, 8W]: decode about four megapixels of output at a time (4 images at 1024 x 1024),
        # so a rollout batch of any size needs a bounded workspace.
        step = max(1, (1 << 22) // max(1, 64 * z.shape[-2] * z.shape[-1]))
        outs = []
        for i in range(0, z.shape[0], step):
            x = self.dec(self.dec_in(z[i : i + step].to(p.dtype)))
            outs.append((self.dec_out(F.silu(self.dec_norm(x))).float() / 2 + 0.5).clamp(0, 1))
        img = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        return img.view(b, -1, *img.shape[1:]) if video else img

    @torch.no_grad()
    def encode(self, images: torch.Tensor) -> torch.Tensor:
        """Pixels in ``[0, 1]`` ``[B, 3, H, W]`` → model latents (posterior mean)."""
        c = self.cfg
        p = next(self.parameters())
        x = self.enc(self.enc_in((images.float() * 2 - 1).to(p.dtype)))
        mean = self.enc_out(F.silu(self.enc_norm(x))).float()[:, : c.latent_channels]
        return (mean - c.shift_factor) * c.scaling_factor


__all__ = ["LatentVAE", "VAEConfig"]
