"""Frozen text encoders for diffusion conditioning, as one configurable native transformer.

``kind="clip"``  causal, learned absolute positions, quick-GELU / GELU MLP, pooled = hidden state at the EOS position
                 (optionally projected) — CLIP-L / CLIP-G text towers; ``penultimate=True`` returns the second-to-last
                 layer's hidden states the way SD3 consumes them.
``kind="t5"``    bidirectional, relative position bias shared by all layers, RMS norms, gated-GELU MLP, no pooled vector —
                 T5-XXL / UMT5 encoders.
``kind="llm"``   causal decoder-only text tower (Qwen-style) whose last hidden states are the conditioning sequence.

Weights are random-init unless a state dict in this module's own key grammar is loaded; the encoders are frozen aux
modules (never sharded, never trained).  Parity: the encoder calls in ``unirl/models/sd3/text_embed.py:51-140``,
``unirl/models/wan21/text_embed.py``, ``unirl/models/qwen_image/text_embed.py``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class TextEncoderConfig:
    kind: str = "clip"
    vocab_size: int = 49408
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    ffn_dim: int = 3072
    max_length: int = 77
    projection_dim: int = 0  # CLIP text projection (0 = return the raw pooled state)
    penultimate: bool = True
    eos_token_id: int = 2
    rel_buckets: int = 32
    rel_max_distance: int = 128
    eps: float = 1e-6
    act: str = "gelu"  # CLIP MLP activation: "gelu" (open_clip bigG) | "quick_gelu" (OpenAI CLIP-L)
    rel_bias_per_layer: bool = False  # UMT5: every layer owns a relative-position table (T5: the first layer's is shared)
    head_dim: int = 0  # 0: hidden_size / num_heads; ByT5 has 6 heads of 64 on a width of 1472

    @classmethod
    def clip_l(cls) -> "TextEncoderConfig":
        return cls("clip", 49408, 768, 12, 12, 3072, 77, 768, eos_token_id=49407, act="quick_gelu")

    @classmethod
    def clip_g(cls) -> "TextEncoderConfig":
        return cls("clip", 49408, 1280, 32, 20, 5120, 77, 1280, eos_token_id=49407)

    @classmethod
    def t5_xxl(cls) -> "TextEncoderConfig":
        return cls("t5", 32128, 4096, 24, 64, 10240, 256, 0, False)

    @classmethod
    def byt5_small(cls) -> "TextEncoderConfig":
        """The byte-level glyph encoder of HunyuanVideo-1.5 (``google/byt5-small`` geometry: bytes + 3 special ids, EOS = 1)."""
        return cls("t5", 384, 1472, 12, 6, 3584, 256, 0, False, eos_token_id=1, head_dim=64)

    @classmethod
    def umt5_xxl(cls) -> "TextEncoderConfig":
        return cls("t5", 256384, 4096, 24, 64, 10240, 512, 0, False, rel_bias_per_layer=True)

    @classmethod
    def tiny(cls, kind: str = "clip", hidden: int = 32, vocab: int = 512, max_length: int = 16) -> "TextEncoderConfig":
        return cls(kind, vocab, hidden, 2, 4, hidden * 2, max_length, hidden if kind == "clip" else 0, kind == "clip")


class _Layer(nn.Module):
    def __init__(self, c: TextEncoderConfig, dtype: Any, device: Any):
        super().__init__()
        h = c.hidden_size
        self.c = c
        norm = (lambda: nn.LayerNorm(h, eps=1e-5, dtype=dtype, device=device)) if c.kind == "clip" else (lambda: nn.RMSNorm(h, eps=c.eps, dtype=dtype, device=device))
        self.norm1, self.norm2 = norm(), norm()
        bias = c.kind == "clip"
        inner = (c.head_dim * c.num_heads) if c.head_dim else h
        self.qkv = nn.Linear(h, 3 * inner, bias=bias, dtype=dtype, device=device)
        self.out = nn.Linear(inner, h, bias=bias, dtype=dtype, device=device)
        self.fc1 = nn.Linear(h, c.ffn_dim * (1 if c.kind == "clip" else 2), bias=bias, dtype=dtype, device=device)
        self.fc2 = nn.Linear(c.ffn_dim, h, bias=bias, dtype=dtype, device=device)
        self.rel_bias = nn.Embedding(c.rel_buckets, c.num_heads, dtype=dtype, device=device) if (c.kind == "t5" and c.rel_bias_per_layer) else None

    def forward(self, x: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        b, l, h = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(b, l, 3, self.c.num_heads, -1).permute(2, 0, 3, 1, 4)
        scale = None if self.c.kind != "t5" else 1.0  # T5 folds the scale into its initialisation
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=scale)
        x = x + self.out(a.transpose(1, 2).reshape(b, l, -1))
        y = self.fc1(self.norm2(x))
        if self.c.kind == "clip":
            y = y * torch.sigmoid(1.702 * y) if self.c.act == "quick_gelu" else F.gelu(y)
        else:
            g, u = y.chunk(2, -1)
            y = F.gelu(g, approximate="tanh") * u
        return x + self.fc2(y)


class TextEncoder(nn.Module):
    def __init__(self, cfg: TextEncoderConfig, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu"):
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.embed = nn.Embedding(cfg.vocab_size, h, dtype=dtype, device=device)
        self.pos = nn.Embedding(cfg.max_length, h, dtype=dtype, device=device) if cfg.kind == "clip" else None
        self.rel_bias = nn.Embedding(cfg.rel_buckets, cfg.num_heads, dtype=dtype, device=device) if (cfg.kind == "t5" and not cfg.rel_bias_per_layer) else None
        self.layers = nn.ModuleList(_Layer(cfg, dtype, device) for _ in range(cfg.num_layers))
        self.final_norm = nn.LayerNorm(h, eps=1e-5, dtype=dtype, device=device) if cfg.kind == "clip" else nn.RMSNorm(h, eps=cfg.eps, dtype=dtype, device=device)
        self.projection = nn.Linear(h, cfg.projection_dim, bias=False, dtype=dtype, device=device) if cfg.projection_dim else None

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "TextEncoder":
        g = torch.Generator(device="cpu").manual_seed(seed)
        for n, p in self.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g).to(p.device))
            elif n.endswith("bias"):
                p.zero_()
            else:  # norm scales
                p.fill_(1.0)
        return self.requires_grad_(False).eval()

    def _t5_bias(self, l: int, device: Any, table: Optional[nn.Embedding] = None) -> torch.Tensor:
        c = self.cfg
        table = table if table is not None else self.rel_bias
        rel = torch.arange(l, device=device)[None, :] - torch.arange(l, device=device)[:, None]
        nb = c.rel_buckets // 2
        ret = (rel > 0).long() * nb
        n = rel.abs()
        exact = nb // 2
        large = exact + (torch.log(n.float().clamp(min=1) / exact) / math.log(c.rel_max_distance / exact) * (nb - exact)).long()
        bucket = ret + torch.where(n < exact, n, large.clamp(max=nb - 1))
        return table(bucket).permute(2, 0, 1)[None]  # [1, heads, L, L]

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``ids [B, L]`` → ``(hidden [B, L, H], pooled [B, P] | None)``."""
        c = self.cfg
        b, l = ids.shape
        x = self.embed(ids)
        if self.pos is not None:
            x = x + self.pos(torch.arange(l, device=ids.device))[None]
        bias = None
        neg = torch.finfo(x.dtype).min
        if c.kind in ("clip", "llm"):
            bias = torch.full((l, l), neg, dtype=x.dtype, device=ids.device).triu(1)[None, None]
        elif c.kind == "t5" and not c.rel_bias_per_layer:
            bias = self._t5_bias(l, ids.device).to(x.dtype)
        pad = None if (mask is None or c.kind != "t5") else (1.0 - mask[:, None, None, :].to(x.dtype)) * neg
        if pad is not None and bias is not None:
            bias = bias + pad
        hidden_states = []
        for layer in self.layers:
            if c.kind == "t5" and c.rel_bias_per_layer:
                bias = self._t5_bias(l, ids.device, layer.rel_bias).to(x.dtype)
                bias = bias if pad is None else bias + pad
            x = layer(x, bias)
            hidden_states.append(x)
        last = self.final_norm(x)
        seq = hidden_states[-2] if (c.penultimate and len(hidden_states) >= 2) else last
        pooled = None
        if c.kind == "clip":
            eos = (ids == c.eos_token_id).int().argmax(-1) if bool((ids == c.eos_token_id).any()) else (mask.long().sum(-1) - 1 if mask is not None else torch.full((b,), l - 1, device=ids.device))
            pooled = last[torch.arange(b, device=ids.device), eos]
            if self.projection is not None:
                pooled = self.projection(pooled)
        return seq, pooled


__all__ = ["TextEncoder", "TextEncoderConfig"]
