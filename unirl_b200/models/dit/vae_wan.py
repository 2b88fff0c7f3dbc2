"""Causal 3-D KL auto-encoder of the WAN 2.1 / WAN 2.2-14B video checkpoints and of Qwen-Image (the same network used on one frame).

Parameter names are the key grammar of the published ``vae`` folders (``AutoencoderKLWan`` / ``AutoencoderKLQwenImage``:
``encoder.down_blocks.N.…`` as one flat list, ``decoder.up_blocks.N.resnets.M`` / ``.upsamplers.0``, ``mid_block.resnets`` /
``.attentions``, RMS norms with a ``gamma``, ``resample.1`` for the spatial convolutions, ``time_conv`` for the temporal ones), so a
checkpoint loads with ``load_state_dict`` and no renaming.

The published implementation streams: the first frame alone, then one latent frame (four pixel frames) at a time, every causal
convolution keeping its last two input frames in a cache.  Every operator of the network is either per frame or causal in time with a
fixed history, so the streamed result is a function of the whole sequence that can be evaluated in one pass, which is what this module
does (a handful of large convolutions per level instead of hundreds of small launches; one sample at a time bounds the workspace):

* a causal convolution is the plain convolution of the sequence padded with two zero frames in front;
* the temporal down-sampling passes frame 0 through and appends the stride-2, un-padded convolution of the whole sequence;
* the temporal up-sampling passes frame 0 through and turns every later frame into two, by a causal convolution over frames 1… (frame
  0 is not in their history) whose doubled channels are interleaved in time.

Latents are normalised per channel with the checkpoint's ``latents_mean`` / ``latents_std`` (model latents = (codec latents − mean) / std),
the codec runs in fp32 and pixels leave in ``[0, 1]``.

Parity: ``unirl/models/wan21/vae.py:48-101``, ``unirl/models/wan21/image_encode.py:55-125``, ``unirl/models/qwen_image/vae.py:36-75``
(which call the diffusers classes named above).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

_WAN_MEAN = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921)
_WAN_STD = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160)


@dataclass
class WanVAEConfig:
    base_dim: int = 96
    z_dim: int = 16
    dim_mult: Tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    attn_scales: Tuple[float, ...] = ()
    temporal_downsample: Tuple[bool, ...] = (False, True, True)
    latents_mean: Tuple[float, ...] = _WAN_MEAN
    latents_std: Tuple[float, ...] = _WAN_STD
    scaling_factor: float = 1.0  # read by callers of the scalar codecs; this codec normalises per channel
    shift_factor: float = 0.0

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "WanVAEConfig":
        z = int(d.get("z_dim", 16))
        return cls(int(d.get("base_dim", 96)), z, tuple(int(m) for m in d.get("dim_mult", (1, 2, 4, 4))), int(d.get("num_res_blocks", 2)),
                   tuple(float(s) for s in d.get("attn_scales", ())), tuple(bool(t) for t in d.get("temperal_downsample", (False, True, True))),
                   tuple(float(v) for v in (d.get("latents_mean") or (0.0,) * z)), tuple(float(v) for v in (d.get("latents_std") or (1.0,) * z)))

    @classmethod
    def tiny(cls, z_dim: int = 4) -> "WanVAEConfig":
        return cls(8, z_dim, (1, 2, 2, 2), 1, (), (False, True, True), tuple(0.1 * i for i in range(z_dim)), tuple(1.0 + 0.25 * i for i in range(z_dim)))

    @property
    def latent_channels(self) -> int:
        return self.z_dim

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.dim_mult) - 1)

    @property
    def temporal_factor(self) -> int:
        return 2 ** sum(bool(t) for t in self.temporal_downsample)



class _CausalConv3d(nn.Conv3d):
    """``nn.Conv3d`` whose time padding sits entirely in front (``2 · p_t`` zero frames), space padding symmetric."""

    def __init__(self, i: int, o: int, kernel: Any, stride: Any = 1, padding: Any = 0):
        super().__init__(i, o, kernel, stride=stride, padding=0)
        p = (padding,) * 3 if isinstance(padding, int) else tuple(padding)
        self._pad = (p[2], p[2], p[1], p[1], 2 * p[0], 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return super().forward(F.pad(x, self._pad) if any(self._pad) else x)


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, images: bool = True):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(dim, *((1, 1) if images else (1, 1, 1))))
        self.scale = dim ** 0.5

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.normalize(x, dim=1) * self.scale * self.gamma


class _Residual(nn.Module):
    def __init__(self, i: int, o: int):
        super().__init__()
        self.norm1, self.conv1 = _RMSNorm(i, images=False), _CausalConv3d(i, o, 3, padding=1)
        self.norm2, self.conv2 = _RMSNorm(o, images=False), _CausalConv3d(o, o, 3, padding=1)
        self.conv_shortcut = _CausalConv3d(i, o, 1) if i != o else nn.Identity()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + self.conv_shortcut(x)


class _Attention(nn.Module):
    """One-head self-attention over the pixels of each frame."""

    def __init__(self, dim: int):
        super().__init__()
        self.norm, self.to_qkv, self.proj = _RMSNorm(dim), nn.Conv2d(dim, 3 * dim, 1), nn.Conv2d(dim, dim, 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, c, t, h, w = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
        q, k, v = self.to_qkv(self.norm(y)).reshape(b * t, 1, 3 * c, h * w).transpose(2, 3).chunk(3, dim=-1)
        y = F.scaled_dot_product_attention(q, k, v).squeeze(1).transpose(1, 2).reshape(b * t, c, h, w)
        return x + self.proj(y).view(b, t, c, h, w).permute(0, 2, 1, 3, 4)


def _per_frame(fn: Any, x: torch.Tensor) -> torch.Tensor:
    b, c, t, h, w = x.shape
    y = fn(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
    return y.view(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)


class _Upsample(nn.Upsample):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return super().forward(x.float()).type_as(x)


class _Resample(nn.Module):
    def __init__(self, dim: int, mode: str):
        super().__init__()
        self.mode = mode
        if mode.startswith("upsample"):
            self.resample = nn.Sequential(_Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"), nn.Conv2d(dim, dim // 2, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = _CausalConv3d(dim, 2 * dim, (3, 1, 1), padding=(1, 0, 0))
        else:
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = _CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.mode == "upsample3d" and x.shape[2] > 1:
            b, c, t, h, w = x.shape
            y = self.time_conv(x[:, :, 1:]).view(b, 2, c, t - 1, h, w)
            x = torch.cat([x[:, :, :1], torch.stack((y[:, 0], y[:, 1]), 3).reshape(b, c, 2 * (t - 1), h, w)], 2)
        x = _per_frame(self.resample, x)
        if self.mode == "downsample3d" and x.shape[2] > 1:
            x = torch.cat([x[:, :, :1], self.time_conv(x)], 2) if x.shape[2] >= 3 else x[:, :, :1]
        return x


class _Mid(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.resnets = nn.ModuleList([_Residual(dim, dim), _Residual(dim, dim)])
        self.attentions = nn.ModuleList([_Attention(dim)])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class _Encoder(nn.Module):
    def __init__(self, c: WanVAEConfig):
        super().__init__()
        dims = [c.base_dim * u for u in (1, *c.dim_mult)]
        self.conv_in = _CausalConv3d(3, dims[0], 3, padding=1)
        blocks: List[nn.Module] = []
        scale = 1.0
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(c.num_res_blocks):
                blocks.append(_Residual(cin, cout))
                if scale in c.attn_scales:
                    blocks.append(_Attention(cout))
                cin = cout
            if i != len(c.dim_mult) - 1:
                blocks.append(_Resample(cout, "downsample3d" if c.temporal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.down_blocks = nn.ModuleList(blocks)
        self.mid_block = _Mid(dims[-1])
        self.norm_out, self.conv_out = _RMSNorm(dims[-1], images=False), _CausalConv3d(dims[-1], 2 * c.z_dim, 3, padding=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.conv_in(x)
        for blk in self.down_blocks:
            x = blk(x)
        return self.conv_out(F.silu(self.norm_out(self.mid_block(x))))


class _UpBlock(nn.Module):
    def __init__(self, i: int, o: int, n: int, mode: Optional[str]):
        super().__init__()
        self.resnets = nn.ModuleList([_Residual(i if j == 0 else o, o) for j in range(n + 1)])
        self.upsamplers = nn.ModuleList([_Resample(o, mode)]) if mode else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for r in self.resnets:
            x = r(x)
        return x if self.upsamplers is None else self.upsamplers[0](x)


class _Decoder(nn.Module):
    def __init__(self, c: WanVAEConfig):
        super().__init__()
        dims = [c.base_dim * u for u in (c.dim_mult[-1], *c.dim_mult[::-1])]
        up_t = tuple(c.temporal_downsample[::-1])
        self.conv_in, self.mid_block = _CausalConv3d(c.z_dim, dims[0], 3, padding=1), _Mid(dims[0])
        blocks = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            mode = None if i == len(c.dim_mult) - 1 else ("upsample3d" if up_t[i] else "upsample2d")
            blocks.append(_UpBlock(cin // 2 if i > 0 else cin, cout, c.num_res_blocks, mode))  # the up-sampler's convolution halved the width
        self.up_blocks = nn.ModuleList(blocks)
        self.norm_out, self.conv_out = _RMSNorm(dims[-1], images=False), _CausalConv3d(dims[-1], 3, 3, padding=1)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        x = self.mid_block(self.conv_in(z))
        for blk in self.up_blocks:
            x = blk(x)
        return self.conv_out(F.silu(self.norm_out(x)))


class AutoencoderKLWan(nn.Module):
    def __init__(self, cfg: WanVAEConfig, device: Any = "cpu", dtype: torch.dtype = torch.float32):
        super().__init__()
        self.cfg = cfg
        self.encoder, self.decoder = _Encoder(cfg), _Decoder(cfg)
        self.quant_conv, self.post_quant_conv = _CausalConv3d(2 * cfg.z_dim, 2 * cfg.z_dim, 1), _CausalConv3d(cfg.z_dim, cfg.z_dim, 1)
        self.to(device=device, dtype=dtype)

    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> "AutoencoderKLWan":
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("gamma"):
                p.copy_(1.0 + 0.1 * torch.empty(p.shape, dtype=torch.float32).normal_(generator=g))
            elif p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, (1.0 / p[0].numel()) ** 0.5, generator=g))
            else:
                p.copy_(0.02 * torch.empty(p.shape, dtype=torch.float32).normal_(generator=g))
        return self.requires_grad_(False).eval()

    @classmethod
    def from_hf(cls, path: str, device: Any = "cpu", dtype: torch.dtype = torch.float32) -> "AutoencoderKLWan":
        """``path``: the ``vae`` folder of a WAN or Qwen-Image checkpoint (``config.json`` + ``*.safetensors``)."""
        from safetensors.torch import load_file

        with open(os.path.join(path, "config.json")) as f:
            vae = cls(WanVAEConfig.from_hf_dict(json.load(f)), device="cpu", dtype=dtype)
        sd: Dict[str, torch.Tensor] = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                sd.update(load_file(os.path.join(path, name)))
        vae.load_state_dict({k: v.to(dtype) for k, v in sd.items()}, strict=True)
        return vae.to(device).requires_grad_(False).eval()

    def _stats(self, like: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        mean = torch.tensor(c.latents_mean, dtype=torch.float32, device=like.device).view(1, c.z_dim, 1, 1, 1)
        std = torch.tensor(c.latents_std, dtype=torch.float32, device=like.device).view(1, c.z_dim, 1, 1, 1)
        return mean, std

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """Model latents → pixels in ``[0, 1]``: ``[B, C, h, w] → [B, 3, 8h, 8w]`` (one frame), ``[B, C, F, h, w] → [B, 4(F−1)+1, 3, 8h, 8w]``."""
        image = latents.dim() == 4
        z = latents.float().unsqueeze(2) if image else latents.float()
        mean, std = self._stats(z)
        p = next(self.parameters())
        outs = []
        for i in range(z.shape[0]):  # one sample at a time: the widest activation is base_dim x frames x H x W
            x = self.decoder(self.post_quant_conv((z[i : i + 1] * std + mean).to(p.dtype)))
            outs.append((x.float().clamp(-1, 1) / 2 + 0.5))
        px = torch.cat(outs, 0)
        return px[:, :, 0] if image else px.permute(0, 2, 1, 3, 4).contiguous()

    @torch.no_grad()
    def encode_video(self, video: torch.Tensor) -> torch.Tensor:
        """Pixels in ``[0, 1]`` ``[B, 3, T, H, W]`` with ``T = 4k + 1`` → model latents ``[B, C, k + 1, H/8, W/8]`` (mode of the posterior)."""
        if (video.shape[2] - 1) % self.cfg.temporal_factor:
            raise ValueError(f"the codec takes 4k + 1 frames, got {video.shape[2]}")
        p = next(self.parameters())
        outs = [self.quant_conv(self.encoder((video[i : i + 1].float() * 2 - 1).to(p.dtype))).float()[:, : self.cfg.z_dim] for i in range(video.shape[0])]
        mu = torch.cat(outs, 0)
        mean, std = self._stats(mu)
        return (mu - mean) / std

    @torch.no_grad()
    def encode(self, images: torch.Tensor) -> torch.Tensor:
        """``[B, 3, H, W]`` in ``[0, 1]`` → ``[B, C, H/8, W/8]``."""
        return self.encode_video(images.unsqueeze(2))[:, :, 0]


def is_wan_vae(vae_dir: str) -> bool:
    """True for a ``vae`` folder whose ``config.json`` names the causal 3-D codec of WAN / Qwen-Image."""
    with open(os.path.join(vae_dir, "config.json")) as f:
        d = json.load(f)
    return d.get("_class_name") in ("AutoencoderKLWan", "AutoencoderKLQwenImage") and not d.get("is_residual", False)


__all__ = ["AutoencoderKLWan", "WanVAEConfig", "is_wan_vae"]
