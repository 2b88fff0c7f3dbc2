"""The KL auto-encoder of the published image checkpoints (SD3 / SD3.5, FLUX-style: 16 latent channels at 1/8 resolution), as a native
module whose parameter names ARE the checkpoint's key grammar, so ``vae/diffusion_pytorch_model.safetensors`` of a diffusers-layout
checkpoint loads with ``load_state_dict`` and no bridge.

Architecture (the published ``AutoencoderKL``): encoder = ``conv_in`` → per level ``layers_per_block`` residual blocks and a stride-2
convolution padded on the right / bottom only → middle (residual, single-head self-attention over the pixels, residual) → group norm, SiLU,
``conv_out`` to mean and log-variance; decoder = ``conv_in`` → middle → per level (deepest first) ``layers_per_block + 1`` residual blocks
and nearest-neighbour ×2 upsampling with a 3×3 convolution → group norm, SiLU, ``conv_out``.  Group norms have 32 groups and eps 1e-6.
Optional 1×1 ``quant_conv`` / ``post_quant_conv`` (older checkpoints).  Same interface as :class:`LatentVAE`: ``decode`` returns pixels
in ``[0, 1]`` in fp32, ``encode`` the scaled posterior mean.

Parity: ``unirl/models/sd3/vae.py:34-56`` (decode in fp32, ``latents / scaling_factor + shift_factor``), which calls the diffusers class.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class KLConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 16
    block_out_channels: Tuple[int, ...] = (128, 256, 512, 512)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    scaling_factor: float = 1.5305
    shift_factor: float = 0.0609
    use_quant_conv: bool = False
    use_post_quant_conv: bool = False
    mid_block_add_attention: bool = True
    temporal_factor: int = 1

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "KLConfig":
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        if "block_out_channels" in kw:
            kw["block_out_channels"] = tuple(int(v) for v in kw["block_out_channels"])
        return cls(**kw)

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.block_out_channels) - 1)


def _norm(c: int, groups: int) -> nn.GroupNorm:
    return nn.GroupNorm(groups, c, eps=1e-6)


class _Resnet(nn.Module):
    def __init__(self, i: int, o: int, groups: int):
        super().__init__()
        self.norm1, self.conv1 = _norm(i, groups), nn.Conv2d(i, o, 3, padding=1)
        self.norm2, self.conv2 = _norm(o, groups), nn.Conv2d(o, o, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(i, o, 1) if i != o else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.conv_shortcut is None else self.conv_shortcut(x))


class _Attention(nn.Module):
    """Single-head self-attention over the ``H·W`` positions, residual."""

    def __init__(self, c: int, groups: int):
        super().__init__()
        self.group_norm = _norm(c, groups)
        self.to_q, self.to_k, self.to_v = nn.Linear(c, c), nn.Linear(c, c), nn.Linear(c, c)
        self.to_out = nn.ModuleList([nn.Linear(c, c)])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, c, h, w = x.shape
        y = self.group_norm(x).view(b, c, h * w).transpose(1, 2)
        a = F.scaled_dot_product_attention(self.to_q(y)[:, None], self.to_k(y)[:, None], self.to_v(y)[:, None])[:, 0]
        return x + self.to_out[0](a).transpose(1, 2).reshape(b, c, h, w)


class _Mid(nn.Module):
    def __init__(self, c: int, groups: int, attention: bool):
        super().__init__()
        self.resnets = nn.ModuleList([_Resnet(c, c, groups), _Resnet(c, c, groups)])
        self.attentions = nn.ModuleList([_Attention(c, groups)] if attention else [])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.resnets[0](x)
        for a in self.attentions:
            x = a(x)
        return self.resnets[1](x)


class _Down(nn.Module):
    def __init__(self, i: int, o: int, n: int, groups: int, down: bool):
        super().__init__()
        self.resnets = nn.ModuleList([_Resnet(i if k == 0 else o, o, groups) for k in range(n)])
        self.downsamplers = nn.ModuleList([_ConvHolder(nn.Conv2d(o, o, 3, stride=2, padding=0))] if down else [])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for r in self.resnets:
            x = r(x)
        for d in self.downsamplers:
            x = d.conv(F.pad(x, (0, 1, 0, 1)))  # one column on the right, one row at the bottom: the published asymmetric padding
        return x


class _Up(nn.Module):
    def __init__(self, i: int, o: int, n: int, groups: int, up: bool):
        super().__init__()
        self.resnets = nn.ModuleList([_Resnet(i if k == 0 else o, o, groups) for k in range(n)])
        self.upsamplers = nn.ModuleList([_ConvHolder(nn.Conv2d(o, o, 3, padding=1))] if up else [])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for r in self.resnets:
            x = r(x)
        for u in self.upsamplers:
            x = u.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))
        return x


class _ConvHolder(nn.Module):
    """``downsamplers.0.conv`` / ``upsamplers.0.conv`` of the key grammar."""

    def __init__(self, conv: nn.Conv2d):
        super().__init__()
        self.conv = conv


class _Encoder(nn.Module):
    def __init__(self, c: KLConfig):
        super().__init__()
        ch, g = c.block_out_channels, c.norm_num_groups
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([_Down(ch[max(i - 1, 0)], ch[i], c.layers_per_block, g, i < len(ch) - 1) for i in range(len(ch))])
        self.mid_block = _Mid(ch[-1], g, c.mid_block_add_attention)
        self.conv_norm_out, self.conv_out = _norm(ch[-1], g), nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.conv_in(x)
        for blk in self.down_blocks:
            x = blk(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class _Decoder(nn.Module):
    def __init__(self, c: KLConfig):
        super().__init__()
        ch, g = tuple(reversed(c.block_out_channels)), c.norm_num_groups
        self.conv_in = nn.Conv2d(c.latent_channels, ch[0], 3, padding=1)
        self.mid_block = _Mid(ch[0], g, c.mid_block_add_attention)
        self.up_blocks = nn.ModuleList([_Up(ch[max(i - 1, 0)], ch[i], c.layers_per_block + 1, g, i < len(ch) - 1) for i in range(len(ch))])
        self.conv_norm_out, self.conv_out = _norm(ch[-1], g), nn.Conv2d(ch[-1], c.out_channels, 3, padding=1)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        x = self.mid_block(self.conv_in(z))
        for blk in self.up_blocks:
            x = blk(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class AutoencoderKL(nn.Module):
    def __init__(self, cfg: KLConfig, device: Any = "cpu", dtype: torch.dtype = torch.float32):
        super().__init__()
        self.cfg = cfg
        self.encoder, self.decoder = _Encoder(cfg), _Decoder(cfg)
        self.quant_conv = nn.Conv2d(2 * cfg.latent_channels, 2 * cfg.latent_channels, 1) if cfg.use_quant_conv else None
        self.post_quant_conv = nn.Conv2d(cfg.latent_channels, cfg.latent_channels, 1) if cfg.use_post_quant_conv else None
        self.to(device=device, dtype=dtype)

    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> "AutoencoderKL":
        g = torch.Generator(device="cpu").manual_seed(seed)
        for p in self.parameters():
            if p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, (1.0 / p[0].numel()) ** 0.5, generator=g).to(p.device, p.dtype))
        return self.requires_grad_(False).eval()

    @classmethod
    def from_hf(cls, path: str, device: Any = "cpu", dtype: torch.dtype = torch.float32) -> "AutoencoderKL":
        """``path``: the ``vae`` folder of a diffusers-layout checkpoint (``config.json`` + ``diffusion_pytorch_model*.safetensors``)."""
        from safetensors.torch import load_file

        with open(os.path.join(path, "config.json")) as f:
            hf = json.load(f)
        sd: Dict[str, torch.Tensor] = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                sd.update(load_file(os.path.join(path, name)))
        if not sd:
            raise FileNotFoundError(f"{path}: no *.safetensors file")
        cfg = KLConfig.from_hf_dict(hf)
        cfg.use_quant_conv, cfg.use_post_quant_conv = "quant_conv.weight" in sd, "post_quant_conv.weight" in sd  # what the file holds decides
        model = cls(cfg, device=device, dtype=dtype)
        sd = {k: (v.reshape(v.shape[0], v.shape[1]) if (".attentions." in k and k.endswith(".weight") and v.dim() == 4) else v) for k, v in sd.items()}  # 1×1-conv form of older files
        sd = {_old_attention_name(k): v for k, v in sd.items()}
        missing, unexpected = model.load_state_dict({k: v.to(dtype) for k, v in sd.items()}, strict=False)
        if missing or unexpected:
            raise KeyError(f"{path}: parameters without a value {list(missing)[:4]}, tensors without a place {list(unexpected)[:4]}")
        return model.requires_grad_(False).eval()

    # ---- LatentVAE interface ----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """Model latents ``[B, C, H, W]`` → pixels in ``[0, 1]`` ``[B, 3, 8H, 8W]`` (fp32), about four output megapixels at a time."""
        c = self.cfg
        p = next(self.parameters())
        z = latents.float() / c.scaling_factor + c.shift_factor
        step = max(1, (1 << 22) // max(1, c.spatial_factor ** 2 * z.shape[-2] * z.shape[-1]))
        outs = []
        for i in range(0, z.shape[0], step):
            zi = z[i : i + step].to(p.dtype)
            if self.post_quant_conv is not None:
                zi = self.post_quant_conv(zi)
            outs.append((self.decoder(zi).float() / 2 + 0.5).clamp(0, 1))
        return outs[0] if len(outs) == 1 else torch.cat(outs, 0)

    @torch.no_grad()
    def encode(self, images: torch.Tensor) -> torch.Tensor:
        """Pixels in ``[0, 1]`` ``[B, 3, H, W]`` → model latents (posterior mean, shifted and scaled)."""
        c = self.cfg
        p = next(self.parameters())
        h = self.encoder((images.float() * 2 - 1).to(p.dtype))
        if self.quant_conv is not None:
            h = self.quant_conv(h)
        return (h.float()[:, : c.latent_channels] - c.shift_factor) * c.scaling_factor


_OLD_ATTENTION = {".query.": ".to_q.", ".key.": ".to_k.", ".value.": ".to_v.", ".proj_attn.": ".to_out.0."}


def _old_attention_name(k: str) -> str:
    """Files written before the attention classes were unified name the projections query / key / value / proj_attn."""
    if ".attentions." in k:
        for old, new in _OLD_ATTENTION.items():
            k = k.replace(old, new)
    return k


__all__ = ["AutoencoderKL", "KLConfig"]
