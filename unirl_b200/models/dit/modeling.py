"""Generic flow-matching diffusion transformer: one implementation, every DiT family a configuration of it.

Three block kinds cover the image / video models the framework trains:

``JointBlock``   two-stream MMDiT block (separate text and latent weights, one joint attention) — SD3 / SD3.5,
                 FLUX double blocks, Qwen-Image, HunyuanVideo double blocks.  Optional second, latent-only attention
                 (SD3.5-Medium "dual attention" layers).
``SingleBlock``  single-stream block over the concatenated ``[text, latent]`` sequence with a fused
                 ``[qkv | mlp-in]`` projection — FLUX / HunyuanVideo single blocks, Z-Image.
``CrossBlock``   latent self-attention + text cross-attention + FFN with a learned per-block modulation table — WAN.

Position information is either an additive 2-D sin-cos table cropped around its centre (SD3) or axial rotary
embeddings over ``(frame, row, column)`` (everything else).  All linears go through ``ops.linear`` (tcgen05 GEMM for
large token counts), adaLN through the fused LayerNorm-modulate kernel, attention through ``ops.attention`` — the
model code holds no device-specific branches.

Sequence parallelism (Ulysses): when ``sp`` is set, every rank holds ``L / P`` latent tokens; attention exchanges
sequence shards for head shards with one all-to-all before and one after the core attention
(``parallel/ulysses.py``).

Reference behaviour covered: the diffusers transformers the reference wraps (``unirl/models/sd3/bundle.py``,
``unirl/models/wan21/diffusion.py:62-158``, ``unirl/models/qwen_image/diffusion.py``, ``unirl/models/flux2_klein/diffusion.py``,
``unirl/models/z_image/diffusion.py``, ``unirl/models/hunyuan_video*/diffusion.py``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from unirl_b200.ops.attention import dense_attention
from unirl_b200.ops.linear import linear
from unirl_b200.ops.norm import layernorm_modulate, rmsnorm
from unirl_b200.train.inject import lora_apply


@dataclass
class DiTConfig:
    name: str = "dit"
    hidden_size: int = 1536
    num_heads: int = 24
    head_dim: int = 64
    in_channels: int = 16
    image_dim: int = 0  # width of an image encoder's tokens read as a second cross-attention context (WAN 2.1 image-to-video: 1280); 0 = none
    out_channels: Optional[int] = None
    patch_size: Tuple[int, int, int] = (1, 2, 2)  # (frames, rows, cols) per token
    num_joint_blocks: int = 24
    num_single_blocks: int = 0
    num_cross_blocks: int = 0
    dual_attention_blocks: Tuple[int, ...] = ()
    text_dim: int = 4096
    pooled_dim: int = 2048  # 0: no pooled-text conditioning
    mlp_ratio: float = 4.0
    ffn_dim: Optional[int] = None  # explicit FFN width (WAN); default hidden · mlp_ratio
    qk_norm: bool = True
    pos_embed: str = "rope"  # "sincos2d" (additive table) | "rope" (axial rotary)
    pos_embed_max_size: int = 192
    pos_embed_base_size: Optional[int] = None  # grid size the sin-cos coordinates are normalised to (SD3: 64); None: unscaled
    rope_axes: Tuple[int, int, int] = (16, 24, 24)  # head_dim split over (frame, row, col); must sum to head_dim
    rope_theta: float = 10000.0
    guidance_embed: bool = False
    time_freq_dim: int = 256
    eps: float = 1e-6
    is_video: bool = False
    vae_scale_factor: int = 8
    vae_temporal_factor: int = 4
    final_text_block: bool = True  # False: the last joint block does not update the text stream (SD3 "context_pre_only")
    qk_norm_scope: str = "head"  # "head": RMS norm per head over head_dim | "full": one RMS norm over the whole projection (WAN)
    text_in_layers: int = 1  # 2: text embedder is Linear -> GELU(tanh) -> Linear (WAN)
    final_modulation: str = "linear"  # "linear": Linear(silu(vec)) -> (shift, scale) | "table": learned [2, h] table + vec (WAN)

    def __post_init__(self) -> None:
        self.patch_size = tuple(int(p) for p in self.patch_size)
        self.rope_axes = tuple(int(a) for a in self.rope_axes)
        self.dual_attention_blocks = tuple(int(i) for i in self.dual_attention_blocks)
        if self.hidden_size != self.num_heads * self.head_dim:
            raise ValueError(f"hidden_size {self.hidden_size} != heads {self.num_heads} x head_dim {self.head_dim}")
        if self.pos_embed == "rope" and sum(self.rope_axes) != self.head_dim:
            raise ValueError(f"rope_axes {self.rope_axes} must sum to head_dim {self.head_dim}")

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.patch_size[0] * self.patch_size[1] * self.patch_size[2]

    @property
    def mlp_dim(self) -> int:
        return int(self.ffn_dim) if self.ffn_dim else int(self.hidden_size * self.mlp_ratio)

    def num_params(self) -> int:
        h, m = self.hidden_size, self.mlp_dim
        joint = 2 * (6 * h * h + 4 * h * h + 2 * h * m)
        single = 3 * h * h + (3 * h + m) * h + (h + m) * h
        cross = 4 * h * h + 4 * h * h + 2 * h * m
        return self.num_joint_blocks * joint + self.num_single_blocks * single + self.num_cross_blocks * cross


# --------------------------------------------------------------------------------------------------- embeddings
def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features of a scalar per sample (fp32), ``[B] → [B, dim]`` (cos first, as in DiT)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], -1)


def sincos_2d_table(dim: int, size: int, device: Any = "cpu", base_size: Optional[int] = None) -> torch.Tensor:
    """``[size, size, dim]`` fixed 2-D sin-cos table as published with SD3: coordinates ``arange(size) * base_size / size`` (``base_size`` is
    the training grid, 64 for the 1024-pixel models; ``None`` leaves them unscaled), the first half of the channels encodes the column and
    the second half the row, each half as ``[sin | cos]`` over ``dim / 4`` frequencies ``10000^(-2 i / (dim / 2))``."""
    half = dim // 2
    omega = 1.0 / (10000 ** (torch.arange(half // 2, dtype=torch.float64) / (half / 2)))
    coord = torch.arange(size, dtype=torch.float64) * ((base_size / size) if base_size else 1.0)
    ang = coord[:, None] * omega[None]
    axis = torch.cat([ang.sin(), ang.cos()], -1)  # [size, dim / 2]
    return torch.cat([axis[None].expand(size, size, -1), axis[:, None].expand(size, size, -1)], -1).float().to(device)


def axial_rope(cfg: DiTConfig, grid: Tuple[int, int, int], device: Any, text_len: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[text_len + F·H·W, head_dim/2]``: text tokens sit at the origin, latent tokens at ``(f, h, w)``."""
    f, h, w = grid
    pos = torch.stack(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(w), indexing="ij"), -1).reshape(-1, 3).float()
    if text_len:
        pos = torch.cat([torch.zeros(text_len, 3), pos])
    parts = []
    for a, d in enumerate(cfg.rope_axes):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        parts.append(pos[:, a : a + 1] * inv[None])
    ang = torch.cat(parts, -1).to(device)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair rotation of ``x [B, L, H, D]`` by per-token angles ``[L, D/2]`` (one kernel each way on CUDA)."""
    if x.is_cuda:
        from unirl_b200.ops.rope import rope_table

        return rope_table(x, cos, sin, True)
    xf = x.float().unflatten(-1, (-1, 2))
    a, b = xf[..., 0], xf[..., 1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2).to(x.dtype)


class _Lin(nn.Module):
    """Weight (+ bias) holder whose matmul goes through the op layer; optional LoRA host.

    ``targets`` names the adapter-addressable row ranges of a fused weight, e.g. a fused QKV projection exposes
    ``{"to_q": (0, h), "to_k": (h, h), "to_v": (2h, h)}`` so recipes keep the per-projection target names.
    """

    def __init__(self, i: int, o: int, bias: bool = True, dtype: Any = None, device: Any = None, targets: Optional[Dict[str, Tuple[int, int]]] = None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None
        self._targets = dict(targets or {})
        # tensor parallelism (sampler only): "col" = this rank keeps the output features ``tp_index`` (rows of the weight, entries of the
        # bias); "row" = it keeps the input features ``tp_index`` (columns) and the partial outputs are summed over the ranks
        self.tp: Optional[Any] = None
        self.tp_mode: Optional[str] = None
        self.tp_index: Optional[torch.Tensor] = None
        self._targets_full: Dict[str, Tuple[int, int]] = {}

    def lora_targets(self) -> Dict[str, Tuple[str, int, int]]:
        return {name: ("weight", off, rows) for name, (off, rows) in self._targets.items()}

    def shard(self, tp: Any, mode: str, index: torch.Tensor) -> None:
        """Keep this rank's slice of the weight in place (``index`` ascending)."""
        with torch.no_grad():
            idx = index.to(self.weight.device)
            self.weight = nn.Parameter(self.weight.data.index_select(0 if mode == "col" else 1, idx).contiguous(), requires_grad=False)
            if mode == "col" and self.bias is not None:
                self.bias = nn.Parameter(self.bias.data.index_select(0, idx).contiguous(), requires_grad=False)
        self.tp, self.tp_mode, self.tp_index = tp, mode, index.cpu()
        self._targets_full = dict(self._targets)
        if mode == "col":  # adapter-addressable row ranges move with the rows that were kept
            kept, off = {}, 0
            for name, (o, rows) in sorted(self._targets.items(), key=lambda kv: kv[1][0]):
                n = int(((self.tp_index >= o) & (self.tp_index < o + rows)).sum())
                kept[name] = (off, n)
                off += n
            self._targets = kept

    def tp_slice(self, leaf: str, t: torch.Tensor) -> torch.Tensor:
        """This rank's part of a full tensor arriving for parameter ``leaf`` (``weight`` / ``bias``) or for an adapter factor
        ``<target>.lora_A`` ``[r, in]`` / ``<target>.lora_B`` ``[rows of the target, r]``."""
        if self.tp_mode is None:
            return t
        idx = self.tp_index.to(t.device)
        if leaf == "weight":
            return t.index_select(0 if self.tp_mode == "col" else 1, idx)
        if leaf == "bias":
            return t.index_select(0, idx) if self.tp_mode == "col" else t
        target, _, factor = leaf.rpartition(".")
        if self.tp_mode == "row":
            return t.index_select(1, idx) if factor == "lora_A" else t
        if factor == "lora_B":
            o, rows = self._targets_full[target]
            return t.index_select(0, idx[(idx >= o) & (idx < o + rows)] - o)
        return t

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = linear(x, self.weight)
        if getattr(self, "_lora_index", None):
            y = lora_apply(self, "weight", x, y)
        if self.tp_mode == "row":
            y = self.tp.reduce(y)
        return y if self.bias is None else y + self.bias


def _heads(x: torch.Tensor, n: int) -> torch.Tensor:
    return x.unflatten(-1, (n, -1))


def _qk_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, tp: Optional[Any] = None) -> torch.Tensor:
    """RMS norm of ``x [..., heads, head_dim]``: per head when ``w`` has ``head_dim`` entries, over all heads jointly when it has ``heads * head_dim``.
    Under tensor parallelism ``x`` holds this rank's heads and ``w`` their scales; a norm over all heads sums its statistic over the ranks."""
    if w is None:
        return x
    if w.numel() != x.shape[-1]:
        if tp is not None and tp.size > 1:
            ss = tp.reduce(x.float().pow(2).sum((-1, -2)))
            r = torch.rsqrt(ss / float(w.numel() * tp.size) + eps)
            return (x.float() * r[..., None, None] * w.float().view(x.shape[-2], x.shape[-1])).to(x.dtype)
        return rmsnorm(x.reshape(-1, w.numel()), w, eps).view_as(x)
    return rmsnorm(x.reshape(-1, x.shape[-1]), w, eps).view_as(x)


def _head_rows(offset: int, heads: int, head_dim: int, tp: Any) -> torch.Tensor:
    """Rows ``offset + [rank · H/P · D, (rank + 1) · H/P · D)``: the heads a tensor-parallel rank owns inside one part of a fused projection."""
    if heads % tp.size:
        raise ValueError(f"{heads} heads do not split over {tp.size} tensor-parallel ranks")
    n = heads // tp.size * head_dim
    return torch.arange(offset + tp.rank * n, offset + (tp.rank + 1) * n)


def _even_rows(offset: int, width: int, tp: Any) -> torch.Tensor:
    if width % tp.size:
        raise ValueError(f"a width of {width} does not split over {tp.size} tensor-parallel ranks")
    n = width // tp.size
    return torch.arange(offset + tp.rank * n, offset + (tp.rank + 1) * n)


def _shard_norm(p: Optional[nn.Parameter], heads: int, head_dim: int, tp: Any) -> Optional[nn.Parameter]:
    """A q / k norm scale over all heads keeps the entries of this rank's heads; a per-head scale is shared and stays whole."""
    if p is None or p.numel() == head_dim:
        return p
    return nn.Parameter(p.data[_head_rows(0, heads, head_dim, tp).to(p.device)].contiguous(), requires_grad=False)


def _qk_norm_param(cfg: "DiTConfig", dtype: Any, device: Any) -> Optional[nn.Parameter]:
    if not cfg.qk_norm:
        return None
    return nn.Parameter(torch.ones(cfg.hidden_size if cfg.qk_norm_scope == "full" else cfg.head_dim, dtype=dtype, device=device))


class _Attn(nn.Module):
    """QKV + per-head RMS q/k norm + output projection for one stream."""

    def __init__(self, cfg: DiTConfig, out_proj: bool = True, dtype: Any = None, device: Any = None, names: Sequence[str] = ("to_q", "to_k", "to_v", "to_out.0")):
        super().__init__()
        h = cfg.hidden_size
        self.qkv = _Lin(h, 3 * h, True, dtype, device, {names[0]: (0, h), names[1]: (h, h), names[2]: (2 * h, h)})
        self.q_norm, self.k_norm = _qk_norm_param(cfg, dtype, device), _qk_norm_param(cfg, dtype, device)
        self.out = _Lin(h, h, True, dtype, device, {names[3]: (0, h)}) if out_proj else None
        self.n, self.eps = cfg.num_heads, cfg.eps
        self.tp: Optional[Any] = None

    def project(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        q, k, v = self.qkv(x).chunk(3, -1)
        return _qk_norm(_heads(q, self.n), self.q_norm, self.eps, self.tp), _qk_norm(_heads(k, self.n), self.k_norm, self.eps, self.tp), _heads(v, self.n)

    def shard(self, tp: Any) -> None:
        """Tensor parallelism over heads: q / k / v rows of this rank's heads, the matching columns of the output projection."""
        h = self.qkv.weight.shape[0] // 3
        d = h // self.n
        self.qkv.shard(tp, "col", torch.cat([_head_rows(o, self.n, d, tp) for o in (0, h, 2 * h)]))
        if self.out is not None:
            self.out.shard(tp, "row", _head_rows(0, self.n, d, tp))
        self.q_norm, self.k_norm = _shard_norm(self.q_norm, self.n, d, tp), _shard_norm(self.k_norm, self.n, d, tp)
        self.n, self.tp = self.n // tp.size, tp


class _MLP(nn.Module):
    def __init__(self, cfg: DiTConfig, dtype: Any = None, device: Any = None, names: Sequence[str] = ("ff.net.0.proj", "ff.net.2")):
        super().__init__()
        self.fc1 = _Lin(cfg.hidden_size, cfg.mlp_dim, True, dtype, device, {names[0]: (0, cfg.mlp_dim)})
        self.fc2 = _Lin(cfg.mlp_dim, cfg.hidden_size, True, dtype, device, {names[1]: (0, cfg.hidden_size)})

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))

    def shard(self, tp: Any) -> None:
        idx = _even_rows(0, self.fc1.weight.shape[0], tp)
        self.fc1.shard(tp, "col", idx)
        self.fc2.shard(tp, "row", idx)


class AttnContext:
    """Per-forward attention geometry: rotary tables, text length, sequence-parallel context."""

    def __init__(self, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], text_len: int, sp: Optional[Any] = None,
                 text_mask: Optional[torch.Tensor] = None):
        self.cos, self.sin, self.text_len, self.sp, self.text_mask = cos, sin, text_len, sp, text_mask
        self.cos_full: Optional[torch.Tensor] = None  # unsharded tables [text + all latent tokens] for attention on head shards
        self.sin_full: Optional[torch.Tensor] = None
        self.image_ctx: Optional[torch.Tensor] = None  # image-encoder tokens at model width, the second context of the cross blocks

    def rope(self, q: torch.Tensor, k: torch.Tensor, offset: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.cos is None:
            return q, k
        c, s = self.cos[offset : offset + q.shape[1]], self.sin[offset : offset + q.shape[1]]
        return apply_rope(q, c, s), apply_rope(k, c, s)

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_text: int = 0) -> torch.Tensor:
        """``[B, L, H, D]`` bidirectional attention; with Ulysses the last ``L − n_text`` tokens are this rank's shard."""
        if self.sp is not None and self.sp.size > 1:
            return self.sp.attention(q, k, v, n_text)
        return dense_attention(q, k, v)

    def fused_sp_attention(self, attn: "_Attn", x: torch.Tensor, text_qkv: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                           rope: bool = True) -> Optional[torch.Tensor]:
        """Sequence-parallel attention of the latent stream ``x [B, l, hidden]`` (already normalised and modulated) with the sequence → head
        exchange done by the QKV projection itself: the GEMM's epilogue stores every head's columns into the rank that owns the head.
        q / k norm and the rotary embedding then run on this rank's heads over the whole sequence.  ``text_qkv``: projected, normalised
        text tokens (replicated, all heads), joined in front.  Returns ``[B, n_text + l, H, D]`` like :meth:`attend`, or None when this
        projection cannot take the fused form (no peer memory, an adapter on the projection, q / k norms of different scopes)."""
        sp = self.sp
        if sp is None or sp.size <= 1 or getattr(attn.qkv, "_lora_index", None):
            return None
        hd = attn.qkv.weight.shape[0] // (3 * attn.n)
        if not sp.can_scatter_project(x, attn.qkv.weight, attn.n):
            return None
        over_heads = attn.q_norm is not None and attn.k_norm is not None and attn.q_norm.numel() == attn.n * hd and attn.k_norm.numel() == attn.n * hd
        if over_heads and not getattr(sp, "fuse_projection_norm_over_heads", False):
            return None
        if over_heads:
            # a norm over all heads of a token (WAN): its statistic comes out of the projection's epilogue, the scaling happens after the exchange
            q, k, v = sp.scatter_project_normed(x, attn.qkv.weight, attn.qkv.bias, attn.q_norm, attn.k_norm, attn.n, attn.eps)
        elif any(w is not None and w.numel() != hd for w in (attn.q_norm, attn.k_norm)):
            return None
        else:
            q, k, v = sp.scatter_project(x, attn.qkv.weight, attn.qkv.bias, attn.n).unbind(0)  # [B, P·l, H/P, D]
            q, k = _qk_norm(q, attn.q_norm, attn.eps), _qk_norm(k, attn.k_norm, attn.eps)
        return self._attend_head_shard(q, k, v, attn.n, text_qkv, rope)

    def _attend_head_shard(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, text_qkv: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                           rope: bool) -> torch.Tensor:
        """Attention on this rank's heads over all tokens (``q, k, v [B, P·l, H/P, D]``, already normalised) with the replicated text tokens'
        heads sliced in front, rotary embedding from the unsharded tables, and the way back to ``[B, n_text + l, H, D]``."""
        sp = self.sp
        nt = 0
        if text_qkv is not None and text_qkv[0].shape[1]:
            nt, hp = text_qkv[0].shape[1], heads // sp.size
            tq, tk, tv = (t[:, :, sp.rank * hp : (sp.rank + 1) * hp] for t in text_qkv)
            q, k, v = torch.cat([tq, q], 1), torch.cat([tk, k], 1), torch.cat([tv, v], 1)
        if rope and self.cos_full is not None:
            off = self.cos_full.shape[0] - q.shape[1]  # tables carry the text rows in front; a latent-only call skips them
            q, k = apply_rope(q, self.cos_full[off:], self.sin_full[off:]), apply_rope(k, self.cos_full[off:], self.sin_full[off:])
        return sp.finish(dense_attention(q, k, v), nt)

    def fused_sp_single(self, blk: "SingleBlock", xn: torch.Tensor, n_text: int) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """Single-stream block under sequence parallelism: ``xn [B, n_text + l, hidden]`` is text (replicated) in front of this rank's latent
        tokens, and ONE projection makes q, k, v and the MLP input.  The latent rows go through the GEMM whose epilogue delivers the head
        columns to their owners and keeps the MLP columns here; the few text rows take the ordinary projection.  Returns the attention
        output ``[B, n_text + l, H, D]`` and the MLP input ``[B, n_text + l, mlp]``, or None when the fused form does not apply."""
        sp, c = self.sp, blk.cfg
        if sp is None or sp.size <= 1 or getattr(blk.in_proj, "_lora_index", None):
            return None
        if any(w is not None and w.numel() != c.head_dim for w in (blk.q_norm, blk.k_norm)):
            return None
        lat = xn[:, n_text:]
        if not sp.can_scatter_project(lat, blk.in_proj.weight, c.num_heads, c.head_dim):
            return None
        qkv, m_lat = sp.scatter_project(lat, blk.in_proj.weight, blk.in_proj.bias, c.num_heads, c.head_dim)
        q, k, v = qkv.unbind(0)
        q, k = _qk_norm(q, blk.q_norm, c.eps), _qk_norm(k, blk.k_norm, c.eps)
        text_qkv, m = None, m_lat
        if n_text:
            tq, tk, tv, m_txt = blk.in_proj(xn[:, :n_text]).split([c.hidden_size, c.hidden_size, c.hidden_size, c.mlp_dim], -1)
            text_qkv = (_qk_norm(_heads(tq, c.num_heads), blk.q_norm, c.eps), _qk_norm(_heads(tk, c.num_heads), blk.k_norm, c.eps), _heads(tv, c.num_heads))
            m = torch.cat([m_txt, m_lat], 1)
        return self._attend_head_shard(q, k, v, c.num_heads, text_qkv, True), m


class JointBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, idx: int, dtype: Any = None, device: Any = None):
        super().__init__()
        h = cfg.hidden_size
        self.cfg, self.idx = cfg, idx
        self.update_text = cfg.final_text_block or idx < cfg.num_joint_blocks - 1
        self.dual = idx in cfg.dual_attention_blocks
        self.img_mod = _Lin(h, (9 if self.dual else 6) * h, True, dtype, device)
        self.txt_mod = _Lin(h, (6 if self.update_text else 2) * h, True, dtype, device)
        self.img_attn = _Attn(cfg, True, dtype, device)
        self.txt_attn = _Attn(cfg, self.update_text, dtype, device, ("add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"))
        self.img_attn2 = _Attn(cfg, True, dtype, device, ("attn2.to_q", "attn2.to_k", "attn2.to_v", "attn2.to_out.0")) if self.dual else None
        self.img_mlp = _MLP(cfg, dtype, device)
        self.txt_mlp = _MLP(cfg, dtype, device, ("ff_context.net.0.proj", "ff_context.net.2")) if self.update_text else None

    def shard(self, tp: Any) -> None:
        for m in (self.img_attn, self.txt_attn, self.img_attn2, self.img_mlp, self.txt_mlp):
            if m is not None:
                m.shard(tp)

    def forward(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor, ctx: AttnContext) -> Tuple[torch.Tensor, torch.Tensor]:
        eps = self.cfg.eps
        im = self.img_mod(F.silu(vec)).chunk(9 if self.dual else 6, -1)
        tm = self.txt_mod(F.silu(vec)).chunk(6 if self.update_text else 2, -1)
        img_n = layernorm_modulate(img, im[0], im[1], eps)
        img_n2 = layernorm_modulate(img, im[6], im[7], eps) if self.dual else None  # both norms see the block input
        txt_n = layernorm_modulate(txt, tm[0], tm[1], eps)
        qt, kt, vt = self.txt_attn.project(txt_n)
        nt = txt.shape[1]
        a = ctx.fused_sp_attention(self.img_attn, img_n, (qt, kt, vt))
        if a is None:
            qi, ki, vi = self.img_attn.project(img_n)
            q, k, v = torch.cat([qt, qi], 1), torch.cat([kt, ki], 1), torch.cat([vt, vi], 1)
            if ctx.cos is not None:
                q, k = ctx.rope(q, k)
            a = ctx.attend(q, k, v, nt)
        a = a.flatten(-2)
        img = img + im[2].unsqueeze(1) * self.img_attn.out(a[:, nt:])
        if self.dual:
            a2 = ctx.fused_sp_attention(self.img_attn2, img_n2, rope=False)
            if a2 is None:
                q2, k2, v2 = self.img_attn2.project(img_n2)
                a2 = ctx.attend(q2, k2, v2, 0)
            img = img + im[8].unsqueeze(1) * self.img_attn2.out(a2.flatten(-2))
        img = img + im[5].unsqueeze(1) * self.img_mlp(layernorm_modulate(img, im[3], im[4], eps))
        if self.update_text:
            txt = txt + tm[2].unsqueeze(1) * self.txt_attn.out(a[:, :nt])
            txt = txt + tm[5].unsqueeze(1) * self.txt_mlp(layernorm_modulate(txt, tm[3], tm[4], eps))
        return img, txt


class SingleBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, idx: int, dtype: Any = None, device: Any = None):
        super().__init__()
        h, m = cfg.hidden_size, cfg.mlp_dim
        self.cfg, self.idx = cfg, idx
        self.mod = _Lin(h, 3 * h, True, dtype, device)
        self.in_proj = _Lin(h, 3 * h + m, True, dtype, device, {"to_q": (0, h), "to_k": (h, h), "to_v": (2 * h, h), "proj_mlp": (3 * h, m)})  # one GEMM
        self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device)) if cfg.qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device)) if cfg.qk_norm else None
        self.out_proj = _Lin(h + m, h, True, dtype, device, {"proj_out": (0, h)})
        self.n, self.hq, self.mq = cfg.num_heads, h, m  # heads, attention width and MLP width held by this rank

    def shard(self, tp: Any) -> None:
        c = self.cfg
        h, m, d = c.hidden_size, c.mlp_dim, c.head_dim
        mlp = _even_rows(0, m, tp)
        self.in_proj.shard(tp, "col", torch.cat([_head_rows(o, c.num_heads, d, tp) for o in (0, h, 2 * h)] + [3 * h + mlp]))
        self.out_proj.shard(tp, "row", torch.cat([_head_rows(0, c.num_heads, d, tp), h + mlp]))
        self.n, self.hq, self.mq = c.num_heads // tp.size, h // tp.size, m // tp.size

    def forward(self, x: torch.Tensor, vec: torch.Tensor, ctx: AttnContext, n_text: int) -> torch.Tensor:
        c = self.cfg
        shift, scale, gate = self.mod(F.silu(vec)).chunk(3, -1)
        xn = layernorm_modulate(x, shift, scale, c.eps)
        fused = ctx.fused_sp_single(self, xn, n_text)
        if fused is not None:
            a, m = fused
        else:
            q, k, v, m = self.in_proj(xn).split([self.hq, self.hq, self.hq, self.mq], -1)
            q, k = _qk_norm(_heads(q, self.n), self.q_norm, c.eps), _qk_norm(_heads(k, self.n), self.k_norm, c.eps)
            q, k = ctx.rope(q, k)
            a = ctx.attend(q, k, _heads(v, self.n), n_text)
        return x + gate.unsqueeze(1) * self.out_proj(torch.cat([a.flatten(-2), F.gelu(m, approximate="tanh")], -1))


class CrossBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, idx: int, dtype: Any = None, device: Any = None):
        super().__init__()
        h = cfg.hidden_size
        self.cfg, self.idx = cfg, idx
        self.modulation = nn.Parameter(torch.zeros(6, h, dtype=dtype, device=device))  # added to the shared time projection
        self.self_attn = _Attn(cfg, True, dtype, device)
        self.cross_q = _Lin(h, h, True, dtype, device, {"attn2.to_q": (0, h)})
        self.cross_kv = _Lin(h, 2 * h, True, dtype, device, {"attn2.to_k": (0, h), "attn2.to_v": (h, h)})
        self.cross_q_norm, self.cross_k_norm = _qk_norm_param(cfg, dtype, device), _qk_norm_param(cfg, dtype, device)
        self.cross_out = _Lin(h, h, True, dtype, device, {"attn2.to_out.0": (0, h)})
        self.cross_norm = nn.LayerNorm(h, eps=cfg.eps, dtype=dtype, device=device)
        if cfg.image_dim:  # keys / values of the image encoder's tokens: their attention output is added to the text's
            self.cross_kv_img = _Lin(h, 2 * h, True, dtype, device, {"attn2.add_k_proj": (0, h), "attn2.add_v_proj": (h, h)})
            self.cross_k_img_norm = _qk_norm_param(cfg, dtype, device)
        else:
            self.cross_kv_img = self.cross_k_img_norm = None
        self.mlp = _MLP(cfg, dtype, device)
        self.n, self.tp = cfg.num_heads, None

    def shard(self, tp: Any) -> None:
        c = self.cfg
        h, d = c.hidden_size, c.head_dim
        self.self_attn.shard(tp)
        self.cross_q.shard(tp, "col", _head_rows(0, c.num_heads, d, tp))
        self.cross_kv.shard(tp, "col", torch.cat([_head_rows(0, c.num_heads, d, tp), _head_rows(h, c.num_heads, d, tp)]))
        self.cross_out.shard(tp, "row", _head_rows(0, c.num_heads, d, tp))
        self.cross_q_norm, self.cross_k_norm = _shard_norm(self.cross_q_norm, c.num_heads, d, tp), _shard_norm(self.cross_k_norm, c.num_heads, d, tp)
        if self.cross_kv_img is not None:
            self.cross_kv_img.shard(tp, "col", torch.cat([_head_rows(0, c.num_heads, d, tp), _head_rows(h, c.num_heads, d, tp)]))
            self.cross_k_img_norm = _shard_norm(self.cross_k_img_norm, c.num_heads, d, tp)
        self.mlp.shard(tp)
        self.n, self.tp = c.num_heads // tp.size, tp

    def forward(self, img: torch.Tensor, txt: torch.Tensor, tproj: torch.Tensor, ctx: AttnContext) -> torch.Tensor:
        c = self.cfg
        m = (tproj.unflatten(-1, (6, -1)) + self.modulation.unsqueeze(0)).unbind(1)
        img_n = layernorm_modulate(img, m[0], m[1], c.eps)
        a = ctx.fused_sp_attention(self.self_attn, img_n)
        if a is None:
            q, k, v = self.self_attn.project(img_n)
            q, k = ctx.rope(q, k)
            a = ctx.attend(q, k, v, 0)
        img = img + m[2].unsqueeze(1) * self.self_attn.out(a.flatten(-2))
        xq = _qk_norm(_heads(self.cross_q(self.cross_norm(img)), self.n), self.cross_q_norm, c.eps, self.tp)
        xk, xv = self.cross_kv(txt).chunk(2, -1)
        xk = _qk_norm(_heads(xk, self.n), self.cross_k_norm, c.eps, self.tp)
        mask = None if ctx.text_mask is None else ctx.text_mask[:, None, None, :].bool()
        a = F.scaled_dot_product_attention(xq.transpose(1, 2), xk.transpose(1, 2), _heads(xv, self.n).transpose(1, 2), attn_mask=mask)
        if self.cross_kv_img is not None and ctx.image_ctx is not None:
            ik, iv = self.cross_kv_img(ctx.image_ctx).chunk(2, -1)
            ik = _qk_norm(_heads(ik, self.n), self.cross_k_img_norm, c.eps, self.tp)
            a = a + F.scaled_dot_product_attention(xq.transpose(1, 2), ik.transpose(1, 2), _heads(iv, self.n).transpose(1, 2))
        img = img + self.cross_out(a.transpose(1, 2).flatten(-2))
        return img + m[5].unsqueeze(1) * self.mlp(layernorm_modulate(img, m[3], m[4], c.eps))


class _ImageEmbedder(nn.Module):
    """Image-encoder tokens → model width: layer norm, two linear layers with a GELU between, layer norm (the ``image_embedder`` of the
    WAN image-to-video checkpoints)."""

    def __init__(self, i: int, o: int, dtype: Any, device: Any):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(i, dtype=dtype, device=device), nn.LayerNorm(o, dtype=dtype, device=device)
        self.fc1, self.fc2 = _Lin(i, i, True, dtype, device), _Lin(i, o, True, dtype, device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.norm2(self.fc2(F.gelu(self.fc1(self.norm1(x)))))


class DiTTransformer(nn.Module):
    """``forward(latents, timestep, text, pooled) → velocity`` with the latents' shape."""

    block_class_names = ("JointBlock", "SingleBlock", "CrossBlock")
    _no_split_modules = ["JointBlock", "SingleBlock", "CrossBlock"]

    def __init__(self, cfg: DiTConfig, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", gradient_checkpointing: bool = False,
                 sp: Optional[Any] = None):
        super().__init__()
        self.cfg, self.sp, self.gradient_checkpointing = cfg, sp, gradient_checkpointing
        self.tp: Optional[Any] = None  # set by apply_tensor_parallel
        self.checkpoint_layers: Optional[int] = None  # recompute only the first N blocks in backward (None = all): 180 GB of HBM holds the rest
        h = cfg.hidden_size
        self.patch_embed = _Lin(cfg.patch_dim, h, True, dtype, device)
        self.time_in = nn.ModuleList([_Lin(cfg.time_freq_dim, h, True, dtype, device), _Lin(h, h, True, dtype, device)])
        self.pooled_in = nn.ModuleList([_Lin(cfg.pooled_dim, h, True, dtype, device), _Lin(h, h, True, dtype, device)]) if cfg.pooled_dim else None
        self.guidance_in = nn.ModuleList([_Lin(cfg.time_freq_dim, h, True, dtype, device), _Lin(h, h, True, dtype, device)]) if cfg.guidance_embed else None
        self.text_in = _Lin(cfg.text_dim, h, True, dtype, device)
        self.text_in2 = _Lin(h, h, True, dtype, device) if cfg.text_in_layers == 2 else None
        self.time_proj = _Lin(h, 6 * h, True, dtype, device) if cfg.num_cross_blocks else None
        self.image_in = _ImageEmbedder(cfg.image_dim, h, dtype, device) if cfg.image_dim else None
        self.joint_blocks = nn.ModuleList(JointBlock(cfg, i, dtype, device) for i in range(cfg.num_joint_blocks))
        self.single_blocks = nn.ModuleList(SingleBlock(cfg, i, dtype, device) for i in range(cfg.num_single_blocks))
        self.cross_blocks = nn.ModuleList(CrossBlock(cfg, i, dtype, device) for i in range(cfg.num_cross_blocks))
        if cfg.final_modulation == "table":
            self.final_mod = None
            self.final_table = nn.Parameter(torch.zeros(2, h, dtype=dtype, device=device))
        else:
            self.final_mod = _Lin(h, 2 * h, True, dtype, device)
        self.final_proj = _Lin(h, (cfg.out_channels or cfg.in_channels) * cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2], True, dtype, device)
        if cfg.pos_embed == "sincos2d":
            self.register_buffer("pos_table", sincos_2d_table(h, cfg.pos_embed_max_size, device, cfg.pos_embed_base_size).to(dtype), persistent=False)
        self._rope_cache: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}

    # ---- init ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "DiTTransformer":
        """Deterministic init; modulation and output projections get a smaller std so a fresh model is near-identity."""
        for i, (name, p) in enumerate(self.named_parameters()):
            if p.dim() < 2:
                if "norm" in name:
                    p.fill_(1.0)
                else:
                    p.zero_()
                continue
            g = torch.Generator(device=p.device)
            g.manual_seed(seed * 100003 + i)
            s = std * (0.25 if any(k in name for k in ("_mod", "mod.", "final_", "modulation")) else 1.0)
            p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, s, generator=g))
        return self

    # ---- patch layout ----------------------------------------------------------------------------------
    def patchify(self, x: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        """``[B, C, (F,) H, W]`` → tokens ``[B, L, C·pf·ph·pw]`` and the token grid."""
        if x.dim() == 4:
            x = x.unsqueeze(2)
        b, c, f, hh, ww = x.shape
        pf, ph, pw = self.cfg.patch_size
        grid = (f // pf, hh // ph, ww // pw)
        x = x.view(b, c, grid[0], pf, grid[1], ph, grid[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(b, grid[0] * grid[1] * grid[2], c * pf * ph * pw), grid

    def unpatchify(self, tokens: torch.Tensor, grid: Tuple[int, int, int], video: bool) -> torch.Tensor:
        b = tokens.shape[0]
        pf, ph, pw = self.cfg.patch_size
        c = tokens.shape[-1] // (pf * ph * pw)
        x = tokens.view(b, grid[0], grid[1], grid[2], c, pf, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        x = x.reshape(b, c, grid[0] * pf, grid[1] * ph, grid[2] * pw)
        return x if video else x.squeeze(2)

    def _pos_crop(self, grid: Tuple[int, int, int]) -> torch.Tensor:
        m = self.cfg.pos_embed_max_size
        top, left = (m - grid[1]) // 2, (m - grid[2]) // 2
        return self.pos_table[top : top + grid[1], left : left + grid[2]].reshape(1, grid[1] * grid[2], -1)

    def _rope(self, grid: Tuple[int, int, int], text_len: int, device: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        key = (grid, text_len, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = axial_rope(self.cfg, grid, device, text_len)
        return self._rope_cache[key]

    # ---- forward ---------------------------------------------------------------------------------------
    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, text: torch.Tensor, pooled: Optional[torch.Tensor] = None,
                text_mask: Optional[torch.Tensor] = None, guidance: Optional[torch.Tensor] = None, image_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg = self.cfg
        video = latents.dim() == 5
        dtype = self.patch_embed.weight.dtype
        tokens, grid = self.patchify(latents.to(dtype))
        img = self.patch_embed(tokens)
        if cfg.pos_embed == "sincos2d":
            img = img + self._pos_crop(grid).to(img.dtype)
        vec = self.time_in[1](F.silu(self.time_in[0](timestep_embedding(timestep, cfg.time_freq_dim).to(dtype))))
        if self.pooled_in is not None and pooled is not None:
            vec = vec + self.pooled_in[1](F.silu(self.pooled_in[0](pooled.to(dtype))))
        if self.guidance_in is not None and guidance is not None:
            vec = vec + self.guidance_in[1](F.silu(self.guidance_in[0](timestep_embedding(guidance, cfg.time_freq_dim).to(dtype))))
        txt = self.text_in(text.to(dtype))
        if self.text_in2 is not None:
            txt = self.text_in2(F.gelu(txt, approximate="tanh"))
        nt = txt.shape[1]
        sp = self.sp if (self.sp is not None and self.sp.size > 1) else None
        if sp is not None:
            img = sp.shard_sequence(img)
        cos = sin = cos_full = sin_full = None
        if cfg.pos_embed == "rope":
            joint_text = nt if (cfg.num_joint_blocks or cfg.num_single_blocks) else 0
            cos, sin = self._rope(grid, joint_text, img.device)
            if sp is not None:
                cos_full, sin_full = cos, sin
                cos, sin = sp.shard_rope(cos, joint_text), sp.shard_rope(sin, joint_text)
        ctx = AttnContext(cos, sin, nt, sp, text_mask)
        ctx.cos_full, ctx.sin_full = cos_full, sin_full
        ctx.image_ctx = self.image_in(image_embeds.to(dtype)) if (self.image_in is not None and image_embeds is not None) else None
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        n_ckpt = None if self.checkpoint_layers is None else int(self.checkpoint_layers)
        done = [0]

        def run(blk: nn.Module, *a: Any):  # blocks are counted in execution order: joint, single, cross
            use = ckpt and (n_ckpt is None or done[0] < n_ckpt)
            done[0] += 1
            return torch.utils.checkpoint.checkpoint(blk, *a, use_reentrant=False) if use else blk(*a)

        for blk in self.joint_blocks:
            img, txt = run(blk, img, txt, vec, ctx)
        if len(self.single_blocks):
            x = torch.cat([txt, img], 1)
            for blk in self.single_blocks:
                x = run(blk, x, vec, ctx, nt)
            img = x[:, nt:]
        if len(self.cross_blocks):
            tproj = self.time_proj(F.silu(vec))
            cross_ctx = AttnContext(cos, sin, 0, sp, text_mask)
            cross_ctx.cos_full, cross_ctx.sin_full, cross_ctx.image_ctx = cos_full, sin_full, ctx.image_ctx
            for blk in self.cross_blocks:
                img = run(blk, img, txt, tproj, cross_ctx)
        if self.final_mod is None:
            shift, scale = (self.final_table.unsqueeze(0) + vec.unsqueeze(1)).unbind(1)
        else:
            shift, scale = self.final_mod(F.silu(vec)).chunk(2, -1)
        out = self.final_proj(layernorm_modulate(img, shift, scale, cfg.eps))
        if sp is not None:
            out = sp.gather_sequence(out)
            sp.end_forward()
        return self.unpatchify(out, grid, video)

    # ---- tensor parallelism (sampler) --------------------------------------------------------------------
    def apply_tensor_parallel(self, tp: Any) -> "DiTTransformer":
        """Shard every block over the heads / MLP width of ``tp`` (``rank``, ``size``, ``reduce``) in place: QKV, the MLP's first layer and
        the cross-attention projections keep this rank's output features, the output projections and the MLP's second layer its input
        features with their partial results summed over the ranks; embedders, modulation layers and the final layer stay whole.
        Inference only.  Call after the full weights are in place; :meth:`tp_slice` cuts tensors that arrive later."""
        if tp is None or tp.size <= 1:
            return self
        if self.sp is not None and getattr(self.sp, "size", 1) > 1:
            raise ValueError("tensor and sequence parallelism of one DiT replica are not combined")
        for blk in [*self.joint_blocks, *self.single_blocks, *self.cross_blocks]:
            blk.shard(tp)
        self.tp = tp
        return self.requires_grad_(False).eval()

    def tp_slice(self, name: str, t: torch.Tensor) -> torch.Tensor:
        """This rank's part of the FULL tensor ``t`` of parameter ``name`` (or of a LoRA factor ``<module>.<target>.lora_{A,B}…``); tensors of
        modules that are not sharded come back whole."""
        if getattr(self, "tp", None) is None:
            return t
        mods = dict(self.named_modules())
        parts = name.split(".")
        for cut in range(len(parts) - 1, 0, -1):
            mod = mods.get(".".join(parts[:cut]))
            if isinstance(mod, _Lin):
                leaf = ".".join(parts[cut:])
                if ".lora_" in "." + leaf:  # "<target>.lora_A.<adapter>.weight" -> "<target>.lora_A"
                    bits = leaf.split(".")
                    k = next(i for i, b in enumerate(bits) if b.startswith("lora_"))
                    leaf = ".".join(bits[: k + 1])
                return mod.tp_slice(leaf, t)
            if isinstance(mod, (_Attn, CrossBlock)) and parts[cut] in ("q_norm", "k_norm", "cross_q_norm", "cross_k_norm") and cut == len(parts) - 1:
                own = getattr(mod, parts[cut])
                if own is not None and own.numel() != t.numel():
                    n_full = (mod.n if isinstance(mod, _Attn) else mod.n) * self.tp.size
                    return t[_head_rows(0, n_full, t.numel() // n_full, self.tp).to(t.device)]
                return t
        return t

    def lora_target_modules(self, patterns: Sequence[str] = ("qkv", "out", "fc1", "fc2", "in_proj", "out_proj", "cross_q", "cross_kv", "cross_out")) -> List[str]:
        """Dotted names of the ``_Lin`` modules a LoRA recipe may wrap (attention and MLP projections inside blocks)."""
        names = []
        for n, m in self.named_modules():
            if isinstance(m, _Lin) and ("blocks." in n) and n.split(".")[-1] in patterns:
                names.append(n)
        return names


__all__ = ["DiTConfig", "DiTTransformer", "JointBlock", "SingleBlock", "CrossBlock", "AttnContext", "timestep_embedding", "sincos_2d_table",
           "axial_rope", "apply_rope"]
