"""Qwen2.5-VL natively: a vision tower whose patch features replace the image placeholder tokens of a Qwen decoder with
3-axis ("multimodal") rotary positions.

Vision tower: flattened ``temporal_patch x patch x patch`` pixel patches → linear patch embedding → ``depth`` pre-norm
blocks (RMSNorm, 2-D rotary attention, SwiGLU MLP) → 2x2 spatial merger MLP into the decoder width.  Patches are reordered
so that each attention window is contiguous: the blocks listed in ``fullatt_block_indexes`` attend over a whole frame, the
others only inside their window (both are packed-sequence boundaries of one varlen attention call); the merger output is put
back into raster order.  Decoder: the Qwen3 decoder class with QKV bias and without QK-norm.

Positions: text tokens advance all three axes together; the ``t·h·w / 4`` placeholder tokens of an image take
``(t, row, col)`` offsets from the image's start position; the text after an image continues from the largest position
used so far + 1.  ``rope_delta = next position − sequence length`` is what decode adds to the cache index.
Parity: the HF ``Qwen2_5_VLForConditionalGeneration`` behaviour relied on by ``unirl/models/qwen_vl/ar.py:28-72, 215-…``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer, TPContext
from unirl_b200.ops.attention import varlen_attention
from unirl_b200.ops.linear import linear
from unirl_b200.ops.norm import rmsnorm


@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 3584
    eps: float = 1e-6
    window_size: int = 112  # pixels; blocks outside `fullatt_block_indexes` attend inside windows of this size
    fullatt_block_indexes: Tuple[int, ...] = (7, 15, 23, 31)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


@dataclass
class QwenVLConfig(Qwen3Config):
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: int = 128
    qk_norm: bool = False
    attention_bias: bool = True
    mrope_section: Tuple[int, int, int] = (16, 24, 24)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision: VisionConfig = field(default_factory=VisionConfig)

    @classmethod
    def qwen25_vl_7b(cls) -> "QwenVLConfig":
        return cls()

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "QwenVLConfig":
        """``config.json`` of a Qwen2.5-VL checkpoint: decoder fields live at the top level (older files) or under
        ``text_config``; the vision tower under ``vision_config``; the rotary sections under ``rope_scaling`` / ``rope_parameters``."""
        text = dict(d.get("text_config") or {})
        flat = {**{k: v for k, v in d.items() if k not in ("text_config", "vision_config")}, **text}
        keys = {f for f in cls.__dataclass_fields__} - {"vision", "mrope_section"}
        kw = {k: v for k, v in flat.items() if k in keys and v is not None}
        rope = flat.get("rope_parameters") or flat.get("rope_scaling") or {}
        if "rope_theta" not in kw and rope.get("rope_theta") is not None:
            kw["rope_theta"] = float(rope["rope_theta"])
        if rope.get("mrope_section"):
            kw["mrope_section"] = tuple(int(v) for v in rope["mrope_section"])
        kw.setdefault("head_dim", kw["hidden_size"] // kw["num_attention_heads"])
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        kw["qk_norm"], kw["attention_bias"] = False, True
        v = dict(d.get("vision_config") or {})
        vkeys = {f for f in VisionConfig.__dataclass_fields__}
        vkw = {k: val for k, val in v.items() if k in vkeys and val is not None}
        if "fullatt_block_indexes" in vkw:
            vkw["fullatt_block_indexes"] = tuple(int(i) for i in vkw["fullatt_block_indexes"])
        if "in_chans" in v and "in_channels" not in vkw:
            vkw["in_channels"] = int(v["in_chans"])
        vkw.setdefault("out_hidden_size", kw["hidden_size"])
        return cls(vision=VisionConfig(**vkw), **kw)

    @classmethod
    def tiny(cls, **kw: Any) -> "QwenVLConfig":
        base = dict(vocab_size=4096, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                    eos_token_id=2, pad_token_id=0, mrope_section=(4, 6, 6), image_token_id=5, video_token_id=6, vision_start_token_id=4,
                    vision=VisionConfig(depth=2, hidden_size=64, num_heads=4, intermediate_size=128, patch_size=4, temporal_patch_size=1, out_hidden_size=128,
                                        window_size=16, fullatt_block_indexes=(1,)))
        base.update(kw)
        return cls(**base)


class _VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype: Any, device: Any):
        super().__init__()
        h = c.hidden_size
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))  # noqa: E731
        self.norm1, self.norm2 = mk(h), mk(h)
        self.qkv, self.qkv_bias = mk(3 * h, h), mk(3 * h)
        self.proj, self.proj_bias = mk(h, h), mk(h)
        self.gate_up, self.gate_up_bias = mk(2 * c.intermediate_size, h), mk(2 * c.intermediate_size)
        self.down, self.down_bias = mk(h, c.intermediate_size), mk(h)
        self.c = c

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, cu: torch.Tensor, max_len: int) -> torch.Tensor:
        c = self.c
        n, d = c.num_heads, c.hidden_size // c.num_heads
        q, k, v = (linear(rmsnorm(x, self.norm1, c.eps), self.qkv) + self.qkv_bias).view(-1, 3, n, d).unbind(1)
        rot = lambda t: (t.float() * cos + torch.cat([-t.float()[..., d // 2 :], t.float()[..., : d // 2]], -1) * sin).to(t.dtype)  # noqa: E731
        a = varlen_attention(rot(q), rot(k), v, cu, max_len, False, d**-0.5)
        x = x + linear(a.reshape(-1, n * d), self.proj) + self.proj_bias
        g, u = (linear(rmsnorm(x, self.norm2, c.eps), self.gate_up) + self.gate_up_bias).chunk(2, -1)
        return x + linear(F.silu(g) * u, self.down) + self.down_bias


class VisionTower(nn.Module):
    def __init__(self, c: VisionConfig, dtype: torch.dtype, device: Any):
        super().__init__()
        self.c = c
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))  # noqa: E731
        self.patch_embed = mk(c.hidden_size, c.patch_dim)
        self.blocks = nn.ModuleList(_VisionBlock(c, dtype, device) for _ in range(c.depth))
        m = c.hidden_size * c.spatial_merge_size**2
        self.merge_norm = mk(c.hidden_size)
        self.merge_fc1, self.merge_fc1_bias = mk(m, m), mk(m)
        self.merge_fc2, self.merge_fc2_bias = mk(c.out_hidden_size, m), mk(c.out_hidden_size)

    def _rope(self, grid_thw: torch.Tensor, device: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        """2-D rotary angles per patch, patches ordered so that each 2x2 merge group is contiguous."""
        c = self.c
        d = c.hidden_size // c.num_heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32) / (d // 2)))
        out = []
        ms = c.spatial_merge_size
        for t, h, w in grid_thw.tolist():
            hh = torch.arange(h).unsqueeze(1).expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            ww = torch.arange(w).unsqueeze(0).expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            ang = torch.cat([hh[:, None] * inv[None], ww[:, None] * inv[None]], -1).repeat(t, 1)
            out.append(ang)
        ang = torch.cat(out).to(device)
        ang = torch.cat([ang, ang], -1)  # half-split rotation convention
        return ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)

    def _windows(self, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Order of the merge groups that makes every attention window contiguous, and the window lengths in patches.
        A window covers ``window_size / patch_size / merge`` merge groups per side; windows at the right / bottom edge are
        partial (an image whose side divides evenly still gets an empty edge window, which is dropped)."""
        c = self.c
        ms, unit = c.spatial_merge_size, c.spatial_merge_size**2
        side = max(c.window_size // ms // c.patch_size, 1)
        order, lens, base = [], [], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // ms, w // ms
            idx = torch.arange(t * gh * gw).view(t, gh, gw)
            ph, pw = side - gh % side, side - gw % side
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (gh + ph) // side, (gw + pw) // side
            idx = idx.view(t, nh, side, nw, side).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, side * side)
            n = (idx >= 0).sum(-1).flatten()
            flat = idx.flatten()
            order.append(flat[flat >= 0] + base)
            lens.append(n[n > 0] * unit)
            base += t * gh * gw
        return torch.cat(order), torch.cat(lens)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``pixel_values [Σ t·h·w, patch_dim]`` (merge-group order), ``grid_thw [n_img, 3]`` → ``[Σ t·h·w / 4, out_hidden]``."""
        c = self.c
        unit = c.spatial_merge_size**2
        x = linear(pixel_values.to(self.patch_embed.dtype), self.patch_embed)
        cos, sin = self._rope(grid_thw, x.device)
        order, win_lens = self._windows(grid_thw)
        order_dev = order.to(x.device)
        regroup = lambda t: t.reshape(-1, unit, *t.shape[1:])[order_dev].reshape(-1, *t.shape[1:])  # noqa: E731
        x, cos, sin = regroup(x), regroup(cos), regroup(sin)
        lens = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])  # full attention stays inside one frame of one image
        cu_full = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32).to(x.device)
        cu_win = F.pad(win_lens.cumsum(0), (1, 0)).to(torch.int32).to(x.device)
        max_full, max_win = int(lens.max()), int(win_lens.max())
        for i, blk in enumerate(self.blocks):
            full = i in c.fullatt_block_indexes
            x = blk(x, cos, sin, cu_full if full else cu_win, max_full if full else max_win)
        x = rmsnorm(x, self.merge_norm, c.eps).view(-1, c.hidden_size * unit)
        x = F.gelu(linear(x, self.merge_fc1) + self.merge_fc1_bias)
        x = linear(x, self.merge_fc2) + self.merge_fc2_bias
        return x[torch.argsort(order).to(x.device)]

    # ---- Hugging Face key grammar (``visual.*``) -------------------------------------------------------------------
    def hf_state_dict(self, prefix: str = "model.visual.") -> Dict[str, torch.Tensor]:
        c, out = self.c, {}
        out[prefix + "patch_embed.proj.weight"] = self.patch_embed.view(c.hidden_size, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size)
        for i, b in enumerate(self.blocks):
            p = f"{prefix}blocks.{i}."
            g, u = b.gate_up.split(c.intermediate_size, 0)
            gb, ub = b.gate_up_bias.split(c.intermediate_size, 0)
            out.update({p + "norm1.weight": b.norm1, p + "norm2.weight": b.norm2, p + "attn.qkv.weight": b.qkv, p + "attn.qkv.bias": b.qkv_bias,
                        p + "attn.proj.weight": b.proj, p + "attn.proj.bias": b.proj_bias, p + "mlp.gate_proj.weight": g, p + "mlp.gate_proj.bias": gb,
                        p + "mlp.up_proj.weight": u, p + "mlp.up_proj.bias": ub, p + "mlp.down_proj.weight": b.down, p + "mlp.down_proj.bias": b.down_bias})
        out.update({prefix + "merger.ln_q.weight": self.merge_norm, prefix + "merger.mlp.0.weight": self.merge_fc1, prefix + "merger.mlp.0.bias": self.merge_fc1_bias,
                    prefix + "merger.mlp.2.weight": self.merge_fc2, prefix + "merger.mlp.2.bias": self.merge_fc2_bias})
        return out

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "model.visual.") -> None:
        self.patch_embed.copy_(sd[prefix + "patch_embed.proj.weight"].reshape(self.patch_embed.shape))
        for i, b in enumerate(self.blocks):
            p = f"{prefix}blocks.{i}."
            b.norm1.copy_(sd[p + "norm1.weight"])
            b.norm2.copy_(sd[p + "norm2.weight"])
            b.qkv.copy_(sd[p + "attn.qkv.weight"])
            b.qkv_bias.copy_(sd[p + "attn.qkv.bias"])
            b.proj.copy_(sd[p + "attn.proj.weight"])
            b.proj_bias.copy_(sd[p + "attn.proj.bias"])
            b.gate_up.copy_(torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]], 0))
            b.gate_up_bias.copy_(torch.cat([sd[p + "mlp.gate_proj.bias"], sd[p + "mlp.up_proj.bias"]], 0))
            b.down.copy_(sd[p + "mlp.down_proj.weight"])
            b.down_bias.copy_(sd[p + "mlp.down_proj.bias"])
        self.merge_norm.copy_(sd[prefix + "merger.ln_q.weight"])
        self.merge_fc1.copy_(sd[prefix + "merger.mlp.0.weight"])
        self.merge_fc1_bias.copy_(sd[prefix + "merger.mlp.0.bias"])
        self.merge_fc2.copy_(sd[prefix + "merger.mlp.2.weight"])
        self.merge_fc2_bias.copy_(sd[prefix + "merger.mlp.2.bias"])


def mrope_positions(tokens: torch.Tensor, grids: Sequence[Sequence[int]], cfg: QwenVLConfig) -> Tuple[torch.Tensor, int]:
    """3-axis positions ``[3, L]`` of one sequence and its ``rope_delta``.  ``grids``: ``(t, h, w)`` per image, in order."""
    ms = cfg.vision.spatial_merge_size
    ids = tokens.tolist()
    pos: List[torch.Tensor] = []
    nxt, i, img = 0, 0, 0
    while i < len(ids):
        if ids[i] in (cfg.image_token_id, cfg.video_token_id) and img < len(grids):
            t, h, w = (int(v) for v in grids[img])
            gh, gw = h // ms, w // ms
            n = t * gh * gw
            tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).flatten()
            hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).flatten()
            ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).flatten()
            pos.append(torch.stack([tt, hh, ww]) + nxt)
            nxt += max(t, gh, gw)
            i += n
            img += 1
        else:
            j = i
            while j < len(ids) and not (ids[j] in (cfg.image_token_id, cfg.video_token_id) and img < len(grids)):
                j += 1
            pos.append((torch.arange(j - i) + nxt).unsqueeze(0).expand(3, -1))
            nxt += j - i
            i = j
    p = torch.cat(pos, 1)[:, : len(ids)] if pos else torch.zeros(3, 0, dtype=torch.long)
    return p, nxt - len(ids)


class QwenVLTransformer(Qwen3Transformer):
    """Decoder + vision tower.  ``forward(tokens, meta)`` as the text model; multimodal prompts go through
    :meth:`prepare_multimodal` first, which fills ``meta.input_embeds`` and 3-axis ``meta.positions``."""

    def __init__(self, cfg: QwenVLConfig, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", tp: Optional[TPContext] = None,
                 gradient_checkpointing: bool = False):
        super().__init__(cfg, dtype, device, tp, gradient_checkpointing)
        self.visual = VisionTower(cfg.vision, dtype, device)

    # ---- Hugging Face key grammar ---------------------------------------------------------------------------------------
    # Two layouts exist: checkpoint files written by older library versions use ``visual.*`` / ``model.layers.*``, newer ones
    # ``model.visual.*`` / ``model.language_model.layers.*``.  Loading accepts both; export writes the newer one.
    @staticmethod
    def _split_hf(sd: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
        text, vis = {}, {}
        for k, v in sd.items():
            if k.startswith("model.visual."):
                vis[k] = v
            elif k.startswith("visual."):
                vis["model." + k] = v
            elif k.startswith("model.language_model."):
                text["model." + k[len("model.language_model."):]] = v
            else:
                text[k] = v
        return text, vis

    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        out = {}
        for k, v in super().hf_state_dict().items():
            out[("model.language_model." + k[len("model."):]) if k.startswith("model.") else k] = v
        out.update(self.visual.hf_state_dict())
        return out

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> None:
        text, vis = self._split_hf(sd)
        super().load_hf_state_dict(text, strict)
        if vis:
            self.visual.load_hf_state_dict(vis)
        elif strict:
            raise KeyError("checkpoint holds no vision tower tensors (visual.* / model.visual.*)")

    def embed_multimodal(self, tokens: torch.Tensor, pixel_values: Optional[torch.Tensor], grid_thw: Optional[torch.Tensor],
                         placeholder_region: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``placeholder_region`` (bool per token): where a placeholder id stands for a vision feature.  A policy may SAMPLE a placeholder id
        in its response; there it is an ordinary token with its text embedding, as it was when the decode step embedded it."""
        x = self.embed_tokens[tokens]
        if pixel_values is None or grid_thw is None or not pixel_values.numel():
            return x
        feats = self.visual(pixel_values.to(x.device), grid_thw.cpu())
        mask = (tokens == self.cfg.image_token_id) | (tokens == self.cfg.video_token_id)
        if placeholder_region is not None:
            mask = mask & placeholder_region.to(mask.device)
        if int(mask.sum()) != feats.shape[0]:
            raise ValueError(f"{int(mask.sum())} image placeholder tokens but {feats.shape[0]} vision features")
        return x.masked_scatter(mask.unsqueeze(-1), feats.to(x.dtype))

    def prepare_multimodal(self, prompts: Sequence[torch.Tensor], extras: Sequence[Any], meta: AttnMeta,
                           prompt_lens: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Packed multimodal prefill / replay set-up.  ``extras[i]``: ``{"pixel_values": [n_i, patch_dim], "image_grid_thw": [k_i, 3]}`` or ``None``.
        ``prompt_lens[i]``: sequence ``i`` is prompt + response and only its first ``prompt_lens[i]`` tokens may hold vision placeholders;
        the response continues the positions one per token (what the decode loop did), whatever ids it contains."""
        dev = self.embed_tokens.device
        pos, deltas, pvs, grids, region = [], [], [], [], []
        for i, (p, e) in enumerate(zip(prompts, extras)):
            g = e.get("image_grid_thw") if e else None
            g = g if g is not None and len(g) else torch.zeros(0, 3, dtype=torch.long)
            n = len(p) if prompt_lens is None else int(prompt_lens[i])
            pp, d = mrope_positions(p[:n].cpu(), g.tolist(), self.cfg)
            if n < len(p):
                tail = torch.arange(n, len(p), dtype=pp.dtype) + int(d)
                pp = torch.cat([pp, tail.unsqueeze(0).expand(pp.shape[0], -1)], 1)
            region.append(torch.arange(len(p)) < n)
            pos.append(pp)
            deltas.append(d)
            if e and e.get("pixel_values") is not None and len(g):
                pvs.append(e["pixel_values"])
                grids.append(torch.as_tensor(g).long())
        tokens = torch.cat([p.to(torch.long) for p in prompts]).to(dev)
        meta.positions = torch.cat(pos, 1).to(dev)
        meta.input_embeds = self.embed_multimodal(tokens, torch.cat(pvs) if pvs else None, torch.cat(grids) if grids else None,
                                                  torch.cat(region) if prompt_lens is not None else None)
        return torch.tensor(deltas, dtype=torch.long)


__all__ = ["QwenVLConfig", "VisionConfig", "VisionTower", "QwenVLTransformer", "mrope_positions"]
