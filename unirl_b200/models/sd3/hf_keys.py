"""Key grammar bridge: a diffusers ``SD3Transformer2DModel`` state dict ↔ the native fused-parameter module.

diffusers keeps separate ``to_q / to_k / to_v`` (and ``add_*_proj``) matrices and ``norm1.linear`` adaLN projections;
the native module fuses QKV per stream and names its modulation ``img_mod / txt_mod``.  ``from_diffusers`` builds
the fused tensors; ``to_diffusers`` splits them again (export and PEFT-compatible LoRA naming).
"""
from __future__ import annotations

from typing import Dict

import torch


def from_diffusers(sd: Dict[str, torch.Tensor], num_blocks: int, dual: tuple = ()) -> Dict[str, torch.Tensor]:
    """diffusers ``SD3Transformer2DModel`` keys → native keys (the shared MMDiT bridge, ``models/dit/hf_keys.py``)."""
    from unirl_b200.models.dit.hf_keys import sd3_from_diffusers

    out = sd3_from_diffusers(sd, num_blocks, dual)
    out.pop("pos_embed_table", None)  # the sin-cos table is recomputed, not stored
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
