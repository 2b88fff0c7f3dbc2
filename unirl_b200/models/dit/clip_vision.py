"""CLIP vision tower: the image encoder of the WAN 2.1 image-to-video checkpoints (ViT-H/14; its penultimate hidden states, one class
token + 256 patch tokens of width 1280, are a second cross-attention context of the transformer).

Pre-norm ViT with a class token and learned absolute positions; pixels are resized to the tower's square input with bicubic
interpolation and normalised with the CLIP statistics, which is what the checkpoint's image processor does to a picture in ``[0, 1]``.

Parity: ``unirl/models/wan21/clip_vision_encode.py:65-83`` (``CLIPVisionModel(..., output_hidden_states=True).hidden_states[-2]``).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

_MEAN = (0.48145466, 0.4578275, 0.40821073)
_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class CLIPVisionConfig:
    hidden_size: int = 1280
    num_layers: int = 32
    num_heads: int = 16
    ffn_dim: int = 5120
    image_size: int = 224
    patch_size: int = 14
    act: str = "gelu"
    eps: float = 1e-5

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "CLIPVisionConfig":
        d = dict(d.get("vision_config") or d)
        return cls(int(d["hidden_size"]), int(d["num_hidden_layers"]), int(d["num_attention_heads"]), int(d["intermediate_size"]), int(d.get("image_size", 224)),
                   int(d.get("patch_size", 14)), str(d.get("hidden_act", "gelu")), float(d.get("layer_norm_eps", 1e-5)))

    @classmethod
    def tiny(cls) -> "CLIPVisionConfig":
        return cls(32, 3, 4, 64, 28, 14, "gelu")

    @property
    def num_tokens(self) -> int:
        return (self.image_size // self.patch_size) ** 2 + 1


class _Layer(nn.Module):
    def __init__(self, c: CLIPVisionConfig, dtype: Any, device: Any):
        super().__init__()
        h = c.hidden_size
        self.c = c
        self.norm1, self.norm2 = nn.LayerNorm(h, eps=c.eps, dtype=dtype, device=device), nn.LayerNorm(h, eps=c.eps, dtype=dtype, device=device)
        self.qkv, self.out = nn.Linear(h, 3 * h, dtype=dtype, device=device), nn.Linear(h, h, dtype=dtype, device=device)
        self.fc1, self.fc2 = nn.Linear(h, c.ffn_dim, dtype=dtype, device=device), nn.Linear(c.ffn_dim, h, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, l, h = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(b, l, 3, self.c.num_heads, -1).permute(2, 0, 3, 1, 4)
        x = x + self.out(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, l, h))
        y = self.fc1(self.norm2(x))
        y = y * torch.sigmoid(1.702 * y) if self.c.act == "quick_gelu" else F.gelu(y)
        return x + self.fc2(y)


class CLIPVisionTower(nn.Module):
    def __init__(self, cfg: CLIPVisionConfig, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu"):
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.class_embedding = nn.Parameter(torch.zeros(h, dtype=dtype, device=device))
        self.patch = nn.Conv2d(3, h, cfg.patch_size, stride=cfg.patch_size, bias=False, dtype=dtype, device=device)
        self.pos = nn.Embedding(cfg.num_tokens, h, dtype=dtype, device=device)
        self.pre_norm = nn.LayerNorm(h, eps=cfg.eps, dtype=dtype, device=device)
        self.layers = nn.ModuleList([_Layer(cfg, dtype, device) for _ in range(cfg.num_layers)])

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "CLIPVisionTower":
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if "norm" in name:
                p.fill_(1.0 if name.endswith("weight") else 0.0)
            else:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g).to(p.dtype))
        return self.requires_grad_(False).eval()

    def preprocess(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[B, 3, H, W]`` in ``[0, 1]`` → the tower's normalised square input."""
        s = self.cfg.image_size
        x = pixels.float()
        if tuple(x.shape[-2:]) != (s, s):
            x = F.interpolate(x, size=(s, s), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
        mean, std = x.new_tensor(_MEAN).view(1, 3, 1, 1), x.new_tensor(_STD).view(1, 3, 1, 1)
        return (x - mean) / std

    @torch.no_grad()
    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """Normalised pixels ``[B, 3, S, S]`` → penultimate hidden states ``[B, 1 + (S / patch)², hidden]``."""
        p = self.patch.weight
        x = self.patch(pixel_values.to(p.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.expand(x.shape[0], 1, -1), x], 1) + self.pos.weight.unsqueeze(0)
        x = self.pre_norm(x)
        for layer in self.layers[:-1]:  # the output of the last layer is never used
            x = layer(x)
        return x

    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        return self.forward(self.preprocess(pixels.to(self.patch.weight.device)))

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> "CLIPVisionTower":
        v = "vision_model."
        own = {"class_embedding": sd[v + "embeddings.class_embedding"], "patch.weight": sd[v + "embeddings.patch_embedding.weight"],
               "pos.weight": sd[v + "embeddings.position_embedding.weight"]}
        for n in ("weight", "bias"):
            own[f"pre_norm.{n}"] = sd[v + f"pre_layrnorm.{n}"]  # the checkpoint's own spelling
        for i in range(self.cfg.num_layers):
            s, d = f"{v}encoder.layers.{i}.", f"layers.{i}."
            for n in ("weight", "bias"):
                own[d + f"qkv.{n}"] = torch.cat([sd[s + f"self_attn.{x}_proj.{n}"] for x in "qkv"], 0)
                own[d + f"out.{n}"] = sd[s + f"self_attn.out_proj.{n}"]
                own[d + f"norm1.{n}"], own[d + f"norm2.{n}"] = sd[s + f"layer_norm1.{n}"], sd[s + f"layer_norm2.{n}"]
                own[d + f"fc1.{n}"], own[d + f"fc2.{n}"] = sd[s + f"mlp.fc1.{n}"], sd[s + f"mlp.fc2.{n}"]
        self.load_state_dict({k: t.to(self.patch.weight.dtype) for k, t in own.items()}, strict=True)
        return self.requires_grad_(False).eval()

    @classmethod
    def from_hf(cls, path: str, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu") -> "CLIPVisionTower":
        """``path``: the ``image_encoder`` folder of a WAN image-to-video checkpoint (``config.json`` + ``*.safetensors``)."""
        from safetensors.torch import load_file

        with open(os.path.join(path, "config.json")) as f:
            tower = cls(CLIPVisionConfig.from_hf_dict(json.load(f)), dtype, device)
        sd: Dict[str, torch.Tensor] = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                sd.update(load_file(os.path.join(path, name)))
        return tower.load_hf_state_dict(sd)


__all__ = ["CLIPVisionConfig", "CLIPVisionTower"]
