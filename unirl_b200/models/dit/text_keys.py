"""Key bridges from Hugging Face text-encoder checkpoints to the native ``TextEncoder``.

``CLIPTextModel`` / ``CLIPTextModelWithProjection`` (the CLIP-L and CLIP-G towers of SD3), ``T5EncoderModel`` (T5-XXL v1.1: gated GELU,
one shared relative-position table) and ``UMT5EncoderModel`` (a table per layer; WAN).  Separate ``q / k / v`` matrices become the fused
``qkv`` weight, ``wi_0 / wi_1`` the fused gate-up weight.  The reference loads these towers through ``transformers`` / diffusers
(``unirl/models/sd3/text_embed.py:51-140``, ``unirl/models/wan21/text_embed.py``); here the published weights go into the native module.
``tests/test_hf_parity_cpu.py`` checks hidden states and pooled vectors against ``transformers`` on small random configurations.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple

import torch

from unirl_b200.models.dit.text_encoder import TextEncoder, TextEncoderConfig

Tensor = torch.Tensor


def config_from_hf(cfg: Dict[str, Any]) -> TextEncoderConfig:
    """``config.json`` of a CLIP text model or a (U)MT5 / T5 encoder → native configuration."""
    mt = str(cfg.get("model_type", "")).lower()
    if "clip" in mt:
        return TextEncoderConfig("clip", int(cfg["vocab_size"]), int(cfg["hidden_size"]), int(cfg["num_hidden_layers"]), int(cfg["num_attention_heads"]),
                                 int(cfg["intermediate_size"]), int(cfg.get("max_position_embeddings", 77)), int(cfg.get("projection_dim", 0) or 0), True,
                                 eos_token_id=int(cfg.get("eos_token_id", 49407)), act=str(cfg.get("hidden_act", "quick_gelu")))
    if "t5" in mt:
        heads, d_kv, d_model = int(cfg["num_heads"]), int(cfg["d_kv"]), int(cfg["d_model"])
        if "gated" not in str(cfg.get("feed_forward_proj", "gated-gelu")):
            raise ValueError("only the gated-GELU T5 variants (v1.1, UMT5) are supported")
        return TextEncoderConfig("t5", int(cfg["vocab_size"]), d_model, int(cfg["num_layers"]), heads, int(cfg["d_ff"]), 512, 0, False,
                                 rel_buckets=int(cfg.get("relative_attention_num_buckets", 32)), rel_max_distance=int(cfg.get("relative_attention_max_distance", 128)),
                                 eps=float(cfg.get("layer_norm_epsilon", 1e-6)), rel_bias_per_layer="umt5" in mt, eos_token_id=int(cfg.get("eos_token_id", 1)),
                                 head_dim=0 if heads * d_kv == d_model else d_kv)
    raise ValueError(f"no text-encoder bridge for model_type {mt!r}")


def clip_text_from_hf(sd: Dict[str, Tensor], num_layers: int) -> Dict[str, Tensor]:
    out: Dict[str, Tensor] = {}
    p = "text_model."
    out["embed.weight"] = sd[p + "embeddings.token_embedding.weight"]
    out["pos.weight"] = sd[p + "embeddings.position_embedding.weight"]
    for i in range(num_layers):
        s, d = f"{p}encoder.layers.{i}.", f"layers.{i}."
        for suf in ("weight", "bias"):
            out[d + "qkv." + suf] = torch.cat([sd[f"{s}self_attn.{n}_proj.{suf}"] for n in ("q", "k", "v")], 0)
            out[d + "out." + suf] = sd[f"{s}self_attn.out_proj.{suf}"]
            out[d + "norm1." + suf] = sd[f"{s}layer_norm1.{suf}"]
            out[d + "norm2." + suf] = sd[f"{s}layer_norm2.{suf}"]
            out[d + "fc1." + suf] = sd[f"{s}mlp.fc1.{suf}"]
            out[d + "fc2." + suf] = sd[f"{s}mlp.fc2.{suf}"]
    out["final_norm.weight"], out["final_norm.bias"] = sd[p + "final_layer_norm.weight"], sd[p + "final_layer_norm.bias"]
    if "text_projection.weight" in sd:
        out["projection.weight"] = sd["text_projection.weight"]
    return out


def t5_from_hf(sd: Dict[str, Tensor], num_layers: int, per_layer_bias: bool) -> Dict[str, Tensor]:
    out: Dict[str, Tensor] = {}
    out["embed.weight"] = sd["shared.weight"] if "shared.weight" in sd else sd["encoder.embed_tokens.weight"]
    for i in range(num_layers):
        s, d = f"encoder.block.{i}.", f"layers.{i}."
        a = s + "layer.0.SelfAttention."
        out[d + "qkv.weight"] = torch.cat([sd[a + "q.weight"], sd[a + "k.weight"], sd[a + "v.weight"]], 0)
        out[d + "out.weight"] = sd[a + "o.weight"]
        out[d + "norm1.weight"] = sd[s + "layer.0.layer_norm.weight"]
        f = s + "layer.1.DenseReluDense."
        out[d + "fc1.weight"] = torch.cat([sd[f + "wi_0.weight"], sd[f + "wi_1.weight"]], 0)  # [gate; up]
        out[d + "fc2.weight"] = sd[f + "wo.weight"]
        out[d + "norm2.weight"] = sd[s + "layer.1.layer_norm.weight"]
        if per_layer_bias:
            out[d + "rel_bias.weight"] = sd[a + "relative_attention_bias.weight"]
    if not per_layer_bias:
        out["rel_bias.weight"] = sd["encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight"]
    out["final_norm.weight"] = sd["encoder.final_layer_norm.weight"]
    return out


_DECODER_TYPES = ("qwen2", "qwen2_vl", "qwen2_5_vl", "qwen3", "llama", "llava", "mistral")


def is_decoder_llm(hf: Dict[str, Any]) -> bool:
    """True for the configuration of a decoder-only language model (possibly inside a vision-language wrapper)."""
    mt = str(hf.get("model_type", "")).lower()
    tmt = str((hf.get("text_config") or {}).get("model_type", "")).lower()
    return mt in _DECODER_TYPES or tmt.replace("_text", "") in _DECODER_TYPES


def load_hf_text_encoder(path: str, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu") -> Tuple[TextEncoder, TextEncoderConfig]:
    """A text-encoder directory in the Hugging Face layout (``config.json`` + ``model*.safetensors``) → a native, frozen ``TextEncoder``."""
    import glob

    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as f:
        hf = json.load(f)
    if is_decoder_llm(hf):  # Qwen2 / Qwen2.5-VL / Qwen3 / LLaMA towers: the package's own decoder behind the encoder interface
        from unirl_b200.models.dit.llm_tower import LLMTextTower

        tower = LLMTextTower.from_hf(path, dtype=dtype, device=device)
        return tower, tower.cfg
    cfg = config_from_hf(hf)
    sd: Dict[str, Tensor] = {}
    for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        sd.update(load_file(fn))
    if not sd:
        raise FileNotFoundError(f"{path}: no *.safetensors shard")
    if cfg.kind == "clip" and "text_projection.weight" not in sd:
        cfg.projection_dim = 0  # a CLIPTextModel without the projection head: the pooled vector is the raw EOS state
    native = clip_text_from_hf(sd, cfg.num_layers) if cfg.kind == "clip" else t5_from_hf(sd, cfg.num_layers, cfg.rel_bias_per_layer)
    enc = TextEncoder(cfg, dtype=dtype, device=device)
    missing, unexpected = enc.load_state_dict({k: v.to(dtype) for k, v in native.items()}, strict=False)
    if missing or unexpected:
        raise KeyError(f"{path}: native parameters without a value {list(missing)[:4]}, checkpoint tensors without a place {list(unexpected)[:4]}")
    return enc.requires_grad_(False).eval(), cfg


__all__ = ["config_from_hf", "clip_text_from_hf", "t5_from_hf", "load_hf_text_encoder", "is_decoder_llm"]
