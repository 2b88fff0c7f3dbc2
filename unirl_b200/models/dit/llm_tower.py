"""Decoder-only language models as frozen text towers of the diffusion families.

Qwen-Image conditions on the last hidden states of Qwen2.5-VL-7B, HunyuanVideo on a LLaMA-3 decoder, Z-Image and FLUX.2 on Qwen3
decoders.  All of them are the decoder this package already trains and serves (``models/qwen3/modeling.py``: grouped-query attention,
rotary positions, SwiGLU, optional q / k norm, optional QKV bias), so the tower is that model behind the encoder interface of
``text_encoder.py`` — ``forward(ids [B, L], mask) → (hidden [B, L, H], None)`` — with its Hugging Face checkpoint importer.

A vision-language checkpoint is read for its language model only: with text-only input the three rotary axes of Qwen2.5-VL carry the
same position, which is the plain rotary embedding, so no vision code is involved.  Padded batches run packed (only real tokens enter the
attention kernel) and come back zero-padded, like the reference's post-processing of its padded encoder output.

Parity: the encoder calls of ``unirl/models/qwen_image/text_embed.py:93-131`` (``Qwen2_5_VLForConditionalGeneration``, last hidden
state) and ``unirl/models/hunyuan_video/text_embed.py`` (LLaMA tower).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer


@dataclass
class LLMTowerInfo:
    """The fields the text-embedding stages read from an encoder's ``cfg``."""

    kind: str
    vocab_size: int
    hidden_size: int
    max_length: int
    eos_token_id: int
    penultimate: bool = False


_BIAS_TYPES = {"qwen2", "qwen2_vl", "qwen2_5_vl", "qwen2_5_vl_text", "qwen2_vl_text"}
_QKNORM_TYPES = {"qwen3"}


def decoder_config_from_hf(d: Dict[str, Any]) -> Qwen3Config:
    """``config.json`` of a Qwen2 / Qwen2.5-VL / Qwen3 / LLaMA checkpoint → the decoder's configuration (the language model's part of a
    vision-language configuration)."""
    text = dict(d.get("text_config") or {})
    merged = {**{k: v for k, v in d.items() if k not in ("text_config", "vision_config")}, **text}
    mt = str(text.get("model_type") or d.get("model_type") or "").lower()
    cfg = Qwen3Config.from_hf_dict(merged)
    cfg.attention_bias = bool(merged.get("attention_bias", mt in _BIAS_TYPES))
    cfg.qk_norm = mt in _QKNORM_TYPES
    cfg.tie_word_embeddings = True  # the tower never projects to the vocabulary: no separate head is kept
    return cfg


def language_model_tensors(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors of the language model under the plain decoder's names (``model.layers.N…``): accepts ``model.language_model.*``
    (newer vision-language files), ``language_model.model.*`` (LLaVA-style wrappers), the plain form and a bare decoder's unprefixed names; vision tensors are dropped."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if ".visual." in "." + k or k.startswith(("vision_tower.", "multi_modal_projector.", "lm_head.")):
            continue
        for old, new in (("model.language_model.", "model."), ("language_model.model.", "model.")):
            if k.startswith(old):
                k = new + k[len(old):]
                break
        if k.startswith(("embed_tokens.", "layers.", "norm.")):
            k = "model." + k  # a bare decoder (``LlamaModel`` / ``Qwen2Model`` saved without the causal-LM wrapper)
        if k.startswith("model."):
            out[k] = v
    return out


class LLMTextTower(nn.Module):
    def __init__(self, cfg: Qwen3Config, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", max_length: int = 1024):
        super().__init__()
        self.decoder = Qwen3Transformer(cfg, dtype=dtype, device=device)
        self.cfg = LLMTowerInfo("llm", cfg.vocab_size, cfg.hidden_size, int(max_length), int(cfg.eos_token_id or 0))

    def init_weights(self, seed: int = 0) -> "LLMTextTower":
        self.decoder.init_weights(seed)
        return self.requires_grad_(False).eval()

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> "LLMTextTower":
        self.decoder.load_hf_state_dict(language_model_tensors(sd), strict=False)
        return self.requires_grad_(False).eval()

    @classmethod
    def from_hf(cls, path: str, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", max_length: int = 1024) -> "LLMTextTower":
        """``path``: a directory with ``config.json`` and ``*.safetensors`` (the ``text_encoder`` folder of a diffusers checkpoint)."""
        from safetensors.torch import load_file

        with open(os.path.join(path, "config.json")) as f:
            tower = cls(decoder_config_from_hf(json.load(f)), dtype, device, max_length)
        sd: Dict[str, torch.Tensor] = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                sd.update(load_file(os.path.join(path, name)))
        return tower.load_hf_state_dict(sd)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, None]:
        """``ids [B, L]`` (right-padded), ``mask [B, L]`` → last hidden states ``[B, L, H]`` after the final norm, zeros at padded positions."""
        b, l = ids.shape
        dev = ids.device
        mask = torch.ones_like(ids) if mask is None else mask.to(dev)
        keep = mask.bool()
        lens = keep.sum(1)
        cu = torch.zeros(b + 1, dtype=torch.int32, device=dev)
        cu[1:] = lens.cumsum(0)
        positions = (keep.long().cumsum(1) - 1)[keep]
        meta = AttnMeta(mode="train", positions=positions, cu_seqlens=cu, max_seqlen=int(lens.max()), seq_lens_host=[int(v) for v in lens.tolist()])
        hidden = self.decoder(ids[keep], meta)
        out = hidden.new_zeros(b, l, hidden.shape[-1])
        out[keep] = hidden
        return out, None


__all__ = ["LLMTextTower", "LLMTowerInfo", "decoder_config_from_hf", "language_model_tensors"]
