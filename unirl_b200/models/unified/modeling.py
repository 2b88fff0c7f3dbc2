"""Unified autoregressive + flow-matching transformer: ONE decoder that writes text token by token and denoises image
latents, with optional mixture-of-experts feed-forward layers.

Two configurations of this module cover the unified families the framework trains:

* HunyuanImage-3 style — sparse MoE FFN (``num_experts`` routed experts, ``experts_per_token`` active, one always-on
  shared expert), the same attention weights for every token.
* Bagel style (mixture of transformers) — two complete parameter sets per layer, hard-routed by modality: text /
  understanding tokens use set 0, generated-image tokens use set 1 (``modality_experts=True``).

Sequence layout in image mode: ``[text tokens | <timestep> | latent patch tokens]``.  Text attends causally; the
timestep and latent tokens attend to the whole text and to each other in both directions.  Rotary positions are 1-D for
text and ``(row, col)`` for latent tokens (half of the rotary frequencies per axis, offset by the text length).

``forward_text(ids, mask)`` → logits-ready hidden states; ``forward_image(ids, mask, latents, t)`` → velocity with the
latents' shape.  Parity: the model-facing behaviour of ``unirl/models/hunyuan_image3/*`` (``mode=gen_text|gen_image``, 4
request modes) and ``unirl/models/bagel/{bundle,diffusion,rl_ops}.py`` (``forward_flow`` with gradients enabled).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from unirl_b200.models.dit.modeling import timestep_embedding
from unirl_b200.ops.linear import linear
from unirl_b200.ops.norm import rmsnorm


@dataclass
class UnifiedConfig:
    name: str = "unified"
    vocab_size: int = 133120
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072  # per expert
    num_experts: int = 64  # 0 = dense FFN
    experts_per_token: int = 8
    shared_expert: bool = True
    modality_experts: bool = False  # mixture of transformers: a second parameter set for generated-image tokens
    latent_channels: int = 32
    patch_size: int = 1
    rope_theta: float = 10000.0
    eps: float = 1e-5
    eos_token_id: int = 2
    pad_token_id: int = 0
    time_freq_dim: int = 256
    router_aux_coef: float = 0.0

    @classmethod
    def hunyuan_image3(cls) -> "UnifiedConfig":
        return cls(name="hunyuan-image3")

    @classmethod
    def bagel_7b(cls) -> "UnifiedConfig":
        return cls(name="bagel-7b", vocab_size=152064, hidden_size=3584, num_layers=28, num_heads=28, num_kv_heads=4, head_dim=128, intermediate_size=18944,
                   num_experts=0, modality_experts=True, latent_channels=16, patch_size=2)

    @classmethod
    def tiny(cls, **kw: Any) -> "UnifiedConfig":
        base = dict(name="tiny-unified", vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=64, num_experts=4,
                    experts_per_token=2, latent_channels=4, patch_size=2)
        base.update(kw)
        return cls(**base)

    @property
    def patch_dim(self) -> int:
        return self.latent_channels * self.patch_size**2


def _p(*shape: int, dtype: Any, device: Any) -> nn.Parameter:
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))


class _FFN(nn.Module):
    def __init__(self, h: int, m: int, dtype: Any, device: Any, tag: str = "mlp"):
        super().__init__()
        self.gate_up, self.down = _p(2 * m, h, dtype=dtype, device=device), _p(h, m, dtype=dtype, device=device)
        self._m, self._h, self._tag = m, h, tag

    def lora_targets(self) -> Dict[str, Tuple[str, int, int]]:
        """``<tag>.gate_proj`` / ``.up_proj`` / ``.down_proj``: ``tag`` is ``mlp`` for the shared / understanding parameters and ``mlp_moe_gen``
        for the generation parameters of a mixture-of-transformers layer (Bagel's adapter targets name them so)."""
        t = self._tag
        return {f"{t}.gate_proj": ("gate_up", 0, self._m), f"{t}.up_proj": ("gate_up", self._m, self._m), f"{t}.down_proj": ("down", 0, self._h)}

    def _proj(self, x: torch.Tensor, name: str) -> torch.Tensor:
        y = linear(x, getattr(self, name))
        if getattr(self, "_lora_index", None):
            from unirl_b200.train.inject import lora_apply

            y = lora_apply(self, name, x, y)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g, u = self._proj(x, "gate_up").chunk(2, -1)
        return self._proj(F.silu(g) * u, "down")


class MoEFFN(nn.Module):
    """Top-k routed experts + optional shared expert.  Tokens are sorted by expert so each expert runs one GEMM pair over its
    contiguous slice; the combine is an index-add weighted by the renormalised router probabilities."""

    def __init__(self, c: UnifiedConfig, dtype: Any, device: Any):
        super().__init__()
        self.c = c
        self.router = _p(c.num_experts, c.hidden_size, dtype=dtype, device=device)
        self.experts = nn.ModuleList(_FFN(c.hidden_size, c.intermediate_size, dtype, device) for _ in range(c.num_experts))
        self.shared = _FFN(c.hidden_size, c.intermediate_size, dtype, device) if c.shared_expert else None
        self.ep: Optional[Any] = None  # ExpertParallelContext once the experts are sharded over a group
        self.expert_ids: List[int] = list(range(c.num_experts))

    def shard_experts(self, ep: Any) -> None:
        """Keep only this rank's experts (``E / P`` consecutive ones); from now on forward dispatches over the expert group."""
        from unirl_b200.parallel.expert_parallel import mark_expert_local

        ids = ep.local_experts(self.c.num_experts)
        self.experts = nn.ModuleList(self.experts[i] for i in ids)
        self.expert_ids, self.ep = ids, ep
        mark_expert_local(self.experts)

    def _forward_ep(self, x: torch.Tensor) -> torch.Tensor:
        c, ep = self.c, self.ep
        xa = ep.gather_tokens(x)  # every rank's tokens, rank-major
        probs = F.softmax(linear(xa, self.router).float(), -1)
        w, idx = probs.topk(c.experts_per_token, -1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        out = torch.zeros_like(xa)
        for slot, e in enumerate(self.expert_ids):
            hit = (idx == e)
            rows = hit.any(-1).nonzero().flatten()
            if rows.numel():
                out.index_add_(0, rows, self.experts[slot](xa[rows]) * (w * hit.to(w.dtype))[rows].sum(-1, keepdim=True))
        y = ep.combine(out)
        return y + self.shared(x) if self.shared is not None else y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.c
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        if self.ep is not None and self.ep.size > 1:
            return self._forward_ep(x).view(shape)
        probs = F.softmax(linear(x, self.router).float(), -1)
        w, idx = probs.topk(c.experts_per_token, -1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        flat_e = idx.flatten()
        order = flat_e.argsort(stable=True)
        tok = torch.arange(x.shape[0], device=x.device).repeat_interleave(c.experts_per_token)[order]
        counts = torch.bincount(flat_e, minlength=c.num_experts).tolist()
        out = torch.zeros_like(x)
        xs, ws = x[tok], w.flatten()[order].unsqueeze(-1)
        start = 0
        for e, n in enumerate(counts):
            if n:
                out.index_add_(0, tok[start : start + n], self.experts[e](xs[start : start + n]) * ws[start : start + n])
            start += n
        if self.shared is not None:
            out = out + self.shared(x)
        return out.view(shape)


def _rope_angles(pos: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=pos.device) / dim))
    return pos.float().unsqueeze(-1) * inv


def _rotate(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """``x [B, L, H, D]``, ``ang [B, L, D/2]`` — half-split convention."""
    h = x.shape[-1] // 2
    c, s = ang.cos().unsqueeze(2), ang.sin().unsqueeze(2)
    x1, x2 = x[..., :h].float(), x[..., h:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


class _ParamSet(nn.Module):
    """Attention + FFN weights of one layer (one set per modality under mixture-of-transformers)."""

    def __init__(self, c: UnifiedConfig, dtype: Any, device: Any, generation: bool = False):
        super().__init__()
        h, d = c.hidden_size, c.head_dim
        self._suffix = "_moe_gen" if generation else ""  # the generation parameter set of a mixture-of-transformers layer
        self.norm1, self.norm2 = _p(h, dtype=dtype, device=device), _p(h, dtype=dtype, device=device)
        self.qkv = _p((c.num_heads + 2 * c.num_kv_heads) * d, h, dtype=dtype, device=device)
        self.q_norm, self.k_norm = _p(d, dtype=dtype, device=device), _p(d, dtype=dtype, device=device)
        self.o = _p(h, c.num_heads * d, dtype=dtype, device=device)
        self.ffn = MoEFFN(c, dtype, device) if c.num_experts else _FFN(h, c.intermediate_size, dtype, device, "mlp_moe_gen" if generation else "mlp")
        self._rows = (c.num_heads * d, c.num_kv_heads * d, h)

    def lora_targets(self) -> Dict[str, Tuple[str, int, int]]:
        """Adapter targets of the attention projections: named row ranges of the fused weights (the unified model is trained with one
        LoRA over its shared backbone, ``unirl/trainer/unified_model.py:133``)."""
        nq, nkv, h = self._rows
        x = self._suffix  # "q_proj" / "q_proj_moe_gen": a recipe may adapt the two parameter sets of a mixture-of-transformers layer separately
        out = {f"q_proj{x}": ("qkv", 0, nq), f"k_proj{x}": ("qkv", nq, nkv), f"v_proj{x}": ("qkv", nq + nkv, nkv), f"o_proj{x}": ("o", 0, h)}
        if not x:
            out["qkv"] = out["qkv_proj"] = ("qkv", 0, nq + 2 * nkv)  # the fused projection under both of its usual names (ask for one)
        return out

    def proj(self, x: torch.Tensor, name: str) -> torch.Tensor:
        y = linear(x, getattr(self, name))
        if getattr(self, "_lora_index", None):
            from unirl_b200.train.inject import lora_apply

            y = lora_apply(self, name, x, y)
        return y


class UnifiedLayer(nn.Module):
    def __init__(self, c: UnifiedConfig, dtype: Any, device: Any):
        super().__init__()
        self.c = c
        self.sets = nn.ModuleList(_ParamSet(c, dtype, device, generation=bool(i)) for i in range(2 if c.modality_experts else 1))

    def _route(self, x: torch.Tensor, gen: Optional[torch.Tensor], fn) -> torch.Tensor:
        """Apply ``fn(param_set, tokens)`` with set 1 on generated-image tokens (``gen`` mask) and set 0 elsewhere."""
        if len(self.sets) == 1 or gen is None or not bool(gen.any()):
            return fn(self.sets[0], x)
        if bool(gen.all()):
            return fn(self.sets[1], x)
        a, b = fn(self.sets[0], x[~gen]), fn(self.sets[1], x[gen])
        out = torch.empty(*x.shape[:-1], a.shape[-1], dtype=a.dtype, device=x.device)
        out[~gen], out[gen] = a, b
        return out

    def forward(self, x: torch.Tensor, ang: torch.Tensor, mask: torch.Tensor, gen: Optional[torch.Tensor], cache: Optional[dict] = None) -> torch.Tensor:
        c = self.c
        b, l, _ = x.shape
        nq, nkv, d = c.num_heads, c.num_kv_heads, c.head_dim
        qkv = self._route(x, gen, lambda s, t: s.proj(rmsnorm(t.reshape(-1, t.shape[-1]), s.norm1, c.eps).view(t.shape), "qkv"))
        q, k, v = qkv.split([nq * d, nkv * d, nkv * d], -1)
        q, k, v = q.view(b, l, nq, d), k.view(b, l, nkv, d), v.view(b, l, nkv, d)
        s0 = self.sets[0]
        q = rmsnorm(q.reshape(-1, d), s0.q_norm, c.eps).view(b, l, nq, d)
        k = rmsnorm(k.reshape(-1, d), s0.k_norm, c.eps).view(b, l, nkv, d)
        q, k = _rotate(q, ang), _rotate(k, ang)
        if cache is not None:  # dense KV cache for the AR loop
            if "k" in cache:
                k, v = torch.cat([cache["k"], k], 1), torch.cat([cache["v"], v], 1)
            cache["k"], cache["v"] = k, v
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask, enable_gqa=nq != nkv)
        a = a.transpose(1, 2).reshape(b, l, nq * d)
        x = x + self._route(a, gen, lambda s, t: s.proj(t, "o"))
        return x + self._route(x, gen, lambda s, t: s.ffn(rmsnorm(t.reshape(-1, t.shape[-1]), s.norm2, c.eps).view(t.shape)))


class UnifiedTransformer(nn.Module):
    block_class_name = "UnifiedLayer"
    _no_split_modules = ["UnifiedLayer"]

    def __init__(self, cfg: UnifiedConfig, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", gradient_checkpointing: bool = False):
        super().__init__()
        self.cfg, self.gradient_checkpointing = cfg, gradient_checkpointing
        h = cfg.hidden_size
        self.embed_tokens = _p(cfg.vocab_size, h, dtype=dtype, device=device)
        self.layers = nn.ModuleList(UnifiedLayer(cfg, dtype, device) for _ in range(cfg.num_layers))
        self.norm = _p(h, dtype=dtype, device=device)
        self.lm_head = _p(cfg.vocab_size, h, dtype=dtype, device=device)
        self.time_in1, self.time_in2 = _p(h, cfg.time_freq_dim, dtype=dtype, device=device), _p(h, h, dtype=dtype, device=device)
        self.patch_in = _p(h, cfg.patch_dim, dtype=dtype, device=device)
        self.patch_out = _p(cfg.patch_dim, h, dtype=dtype, device=device)

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "UnifiedTransformer":
        for i, (n, p) in enumerate(self.named_parameters()):
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                g = torch.Generator(device=p.device)
                g.manual_seed(seed * 100003 + i)
                p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std * (0.25 if n == "patch_out" else 1.0), generator=g))
        return self

    @property
    def output_weight(self) -> torch.Tensor:
        return self.lm_head

    def _run(self, x: torch.Tensor, ang: torch.Tensor, mask: torch.Tensor, gen: Optional[torch.Tensor], caches: Optional[List[dict]] = None) -> torch.Tensor:
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled() and caches is None
        for i, layer in enumerate(self.layers):
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(layer, x, ang, mask, gen, use_reentrant=False)
            else:
                x = layer(x, ang, mask, gen, None if caches is None else caches[i])
        return rmsnorm(x.reshape(-1, x.shape[-1]), self.norm, self.cfg.eps).view(x.shape)

    # ---- text mode ----------------------------------------------------------------------------------------
    def forward_text(self, ids: torch.Tensor, attn_mask: torch.Tensor, caches: Optional[List[dict]] = None, positions: Optional[torch.Tensor] = None,
                     key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``ids [B, L]`` (right-padded) → hidden ``[B, L, H]``; causal, padding keys masked.  With ``caches`` the call is one
        step of incremental decoding (``positions [B, L]`` absolute, ``key_mask [B, L_total]``)."""
        c = self.cfg
        b, l = ids.shape
        pos = positions if positions is not None else torch.arange(l, device=ids.device).expand(b, l)
        ang = torch.cat([_rope_angles(pos, c.head_dim // 2, c.rope_theta)] * 2, -1)
        keys = attn_mask if key_mask is None else key_mask
        lk = keys.shape[1]
        causal = torch.ones(l, lk, dtype=torch.bool, device=ids.device).tril(lk - l)
        mask = causal[None, None] & keys[:, None, None, :].bool()
        return self._run(self.embed_tokens[ids], ang, mask, None, caches)

    # ---- image mode ---------------------------------------------------------------------------------------
    def forward_image(self, ids: torch.Tensor, attn_mask: torch.Tensor, latents: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        """``latents [B, C, H, W]`` at noise level ``timestep [B]`` (0…1000), conditioned on text ``ids [B, L]`` → velocity."""
        c = self.cfg
        b, l = ids.shape
        ch, hh, ww = latents.shape[1:]
        p = c.patch_size
        gh, gw = hh // p, ww // p
        dtype = self.embed_tokens.dtype
        tok = latents.to(dtype).view(b, ch, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(b, gh * gw, ch * p * p)
        temb = linear(F.silu(linear(timestep_embedding(timestep, c.time_freq_dim).to(dtype), self.time_in1)), self.time_in2)
        x = torch.cat([self.embed_tokens[ids], temb.unsqueeze(1), linear(tok, self.patch_in)], 1)
        n_img = 1 + gh * gw
        # positions: text 0..L-1 on both axes; image tokens (row, col) offset by L
        tpos = torch.arange(l, device=ids.device)
        rows = torch.cat([tpos, torch.full((1,), l, device=ids.device), l + 1 + torch.arange(gh, device=ids.device).repeat_interleave(gw)])
        cols = torch.cat([tpos, torch.full((1,), l, device=ids.device), l + 1 + torch.arange(gw, device=ids.device).repeat(gh)])
        ang = torch.cat([_rope_angles(rows, c.head_dim // 2, c.rope_theta), _rope_angles(cols, c.head_dim // 2, c.rope_theta)], -1)
        ang = ang.unsqueeze(0).expand(b, -1, -1)  # [B, L + 1 + gh·gw, head_dim / 2]: half of the frequencies per axis
        total = l + n_img
        mask = torch.zeros(total, total, dtype=torch.bool, device=ids.device)
        mask[:l, :l] = torch.ones(l, l, dtype=torch.bool, device=ids.device).tril()
        mask[l:, :] = True
        keys = torch.cat([attn_mask.bool(), torch.ones(b, n_img, dtype=torch.bool, device=ids.device)], 1)
        mask = mask[None, None] & keys[:, None, None, :]
        gen = torch.zeros(b, total, dtype=torch.bool, device=ids.device)
        gen[:, l:] = True
        h = self._run(x, ang, mask, gen if c.modality_experts else None)
        v = linear(h[:, l + 1 :], self.patch_out)
        return v.view(b, gh, gw, ch, p, p).permute(0, 3, 1, 4, 2, 5).reshape(b, ch, hh, ww)


__all__ = ["UnifiedConfig", "UnifiedTransformer", "UnifiedLayer", "MoEFFN"]
