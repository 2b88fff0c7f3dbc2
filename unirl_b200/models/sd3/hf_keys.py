"""Key grammar bridge: a diffusers ``SD3Transformer2DModel`` state dict ↔ the native fused-parameter module.

diffusers keeps separate ``to_q / to_k / to_v`` (and ``add_*_proj``) matrices and ``norm1.linear`` adaLN projections;
the native module fuses QKV per stream and names its modulation ``img_mod / txt_mod``.  ``from_diffusers`` builds
the fused tensors; ``to_diffusers`` splits them again (export and PEFT-compatible LoRA naming).
"""
from __future__ import annotations

from typing import Dict

import torch


def _cat(sd: Dict[str, torch.Tensor], keys, suffix: str) -> torch.Tensor:
    return torch.cat([sd[f"{k}.{suffix}"] for k in keys], 0)


def from_diffusers(sd: Dict[str, torch.Tensor], num_blocks: int, dual: tuple = ()) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    def put(dst: str, src: str) -> None:
        for s in ("weight", "bias"):
            if f"{src}.{s}" in sd:
                out[f"{dst}.{s}"] = sd[f"{src}.{s}"]
    put("patch_embed", "pos_embed.proj")  # conv [h, c, p, p] is reshaped by the caller to [h, c*p*p]
    if "patch_embed.weight" in out and out["patch_embed.weight"].dim() == 4:
        out["patch_embed.weight"] = out["patch_embed.weight"].flatten(1)
    put("time_in.0", "time_text_embed.timestep_embedder.linear_1"); put("time_in.1", "time_text_embed.timestep_embedder.linear_2")
    put("pooled_in.0", "time_text_embed.text_embedder.linear_1"); put("pooled_in.1", "time_text_embed.text_embedder.linear_2")
    put("text_in", "context_embedder"); put("final_mod", "norm_out.linear"); put("final_proj", "proj_out")
    for i in range(num_blocks):
        s, d = f"transformer_blocks.{i}", f"joint_blocks.{i}"
        put(f"{d}.img_mod", f"{s}.norm1.linear"); put(f"{d}.txt_mod", f"{s}.norm1_context.linear")
        for suf in ("weight", "bias"):
            out[f"{d}.img_attn.qkv.{suf}"] = _cat(sd, [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v"], suf)
            out[f"{d}.txt_attn.qkv.{suf}"] = _cat(sd, [f"{s}.attn.add_q_proj", f"{s}.attn.add_k_proj", f"{s}.attn.add_v_proj"], suf)
            if i in dual:
                out[f"{d}.img_attn2.qkv.{suf}"] = _cat(sd, [f"{s}.attn2.to_q", f"{s}.attn2.to_k", f"{s}.attn2.to_v"], suf)
        put(f"{d}.img_attn.out", f"{s}.attn.to_out.0"); put(f"{d}.txt_attn.out", f"{s}.attn.to_add_out")
        if i in dual:
            put(f"{d}.img_attn2.out", f"{s}.attn2.to_out.0")
        for a, b in (("img_attn.q_norm", "attn.norm_q.weight"), ("img_attn.k_norm", "attn.norm_k.weight"), ("txt_attn.q_norm", "attn.norm_added_q.weight"),
                     ("txt_attn.k_norm", "attn.norm_added_k.weight"), ("img_attn2.q_norm", "attn2.norm_q.weight"), ("img_attn2.k_norm", "attn2.norm_k.weight")):
            if f"{s}.{b}" in sd:
                out[f"{d}.{a}"] = sd[f"{s}.{b}"]
        put(f"{d}.img_mlp.fc1", f"{s}.ff.net.0.proj"); put(f"{d}.img_mlp.fc2", f"{s}.ff.net.2")
        put(f"{d}.txt_mlp.fc1", f"{s}.ff_context.net.0.proj"); put(f"{d}.txt_mlp.fc2", f"{s}.ff_context.net.2")
    return out


def to_diffusers(sd: Dict[str, torch.Tensor], num_blocks: int, hidden: int) -> Dict[str, torch.Tensor]:
    """Inverse of :func:`from_diffusers` for the block weights (used by the HF exporter)."""
    out: Dict[str, torch.Tensor] = {}
    for i in range(num_blocks):
        s, d = f"joint_blocks.{i}", f"transformer_blocks.{i}"
        for suf in ("weight", "bias"):
            for stream, names in (("img_attn", ("attn.to_q", "attn.to_k", "attn.to_v")), ("txt_attn", ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj")),
                                  ("img_attn2", ("attn2.to_q", "attn2.to_k", "attn2.to_v"))):
                key = f"{s}.{stream}.qkv.{suf}"
                if key in sd:
                    for j, n in enumerate(names):
                        out[f"{d}.{n}.{suf}"] = sd[key][j * hidden : (j + 1) * hidden]
    return out


__all__ = ["from_diffusers", "to_diffusers"]
