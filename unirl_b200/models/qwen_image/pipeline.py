"""Qwen-Image: 60 joint blocks, packed 2x2 latents, LLM text tower, dynamic shift, CFG norm correction — config, bundle and pipeline on the generic DiT core.

What the family changes (``unirl/models/qwen_image/text_embed.py:36-131``, ``diffusion.py``):

* **text conditioning**: the prompt is wrapped in a chat template and run through a decoder-only language model (Qwen2.5-VL's); the
  conditioning sequence is the last hidden state WITHOUT the template's system prefix (34 tokens with the published tokenizer), padded
  with zero rows to the longest prompt of the batch, with a mask of the real positions; there is no pooled vector;
* **guidance**: the guided prediction is rescaled, token by token, to the norm of the conditional one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.dit.text_embed import TextEmbedStage
from unirl_b200.types.conditions import TextEmbedCondition
from unirl_b200.types.primitives import Texts

PROMPT_PREFIX = ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, spatial relationships of the objects and background:"
                 "<|im_end|>\n<|im_start|>user\n")
PROMPT_SUFFIX = "<|im_end|>\n<|im_start|>assistant\n"
TOKENIZER_MAX_LENGTH = 1024


@dataclass
class QwenImagePipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:qwen-image"
    use_prompt_template: bool = True


class QwenImageBundle(DiTBundle):
    pass


class QwenImageTextEmbedStage(TextEmbedStage):
    """Chat-templated prompt → language-model hidden states, system prefix cut off, zero-padded to the batch maximum with a mask.
    ``prefix`` / ``suffix`` / ``token_cap`` are class attributes so that a family with another template derives from this stage."""

    prefix, suffix, token_cap = PROMPT_PREFIX, PROMPT_SUFFIX, TOKENIZER_MAX_LENGTH

    def __init__(self, *a: Any, use_template: bool = True, **k: Any):
        super().__init__(*a, **k)
        if self.max_sequence_length > self.token_cap:
            raise ValueError(f"max_sequence_length cannot exceed {self.token_cap} (the tokenizer's cap), got {self.max_sequence_length}")
        self.use_template = bool(use_template)

    @torch.no_grad()
    def embed(self, texts: Any) -> TextEmbedCondition:
        strs: List[str] = [t.to_str() if hasattr(t, "to_str") else str(t) for t in (texts.to_list() if isinstance(texts, Texts) else texts)]
        if not self.use_template:
            return super().embed(strs)
        enc, tok = self.encoders[0], self.tokenizers[0]
        c = enc.cfg
        dev = next(enc.parameters()).device
        crop = len(tok.encode(self.prefix))  # Qwen-Image: 34 with the published tokenizer
        uniq: Dict[str, int] = {}
        for s in strs:
            uniq.setdefault(s, len(uniq))
        rows = [[int(i) % c.vocab_size for i in tok.encode(self.prefix + (s or " ") + self.suffix)][: self.token_cap + crop] for s in uniq]
        width = max(len(r) for r in rows)
        ids = torch.zeros(len(rows), width, dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : len(r)] = torch.tensor(r)
            mask[i, : len(r)] = 1
        seq, _ = enc(ids.to(dev), mask.to(dev))
        mask = mask.to(dev)
        seq = (seq * mask.unsqueeze(-1).to(seq.dtype))[:, crop : crop + self.max_sequence_length]  # zero rows at the padding, whatever the tower returns there
        mask = mask[:, crop : crop + self.max_sequence_length]
        if self.text_dim and seq.shape[-1] != self.text_dim:
            seq = torch.nn.functional.pad(seq, (0, self.text_dim - seq.shape[-1])) if seq.shape[-1] < self.text_dim else seq[..., : self.text_dim]
        idx = torch.tensor([uniq[s] for s in strs], device=seq.device)
        return TextEmbedCondition(embeds=seq[idx], pooled=None, attn_mask=mask[idx])


class QwenImageDiffusionStage(DiTDiffusionStage):
    """CFG with norm correction: the guided prediction is rescaled to the norm of the conditional one (per token)."""

    def _guided(self, v_uncond, v_cond, p):
        vg = v_uncond + p.guidance_scale * (v_cond - v_uncond)
        nc, ng = v_cond.norm(dim=1, keepdim=True), vg.norm(dim=1, keepdim=True).clamp_min(1e-12)
        return vg * (nc / ng)


class QwenImagePipeline(DiTPipeline):
    def __init__(self, bundle, **options):
        super().__init__(bundle, **options)
        spec, cfg = bundle.spec, bundle.config
        self.diffusion = QwenImageDiffusionStage(bundle, spec.default_strategy, cfg.autocast_precision)
        self.text_embed = QwenImageTextEmbedStage(bundle.text_encoders, bundle.tokenizers, spec.text_combine, spec.transformer.text_dim, cfg.max_sequence_length,
                                                  use_template=bool(getattr(cfg, "use_prompt_template", True)))

    @classmethod
    def from_config(cls, config: QwenImagePipelineConfig) -> "QwenImagePipeline":
        return cls(QwenImageBundle.from_config(config))


__all__ = ["QwenImagePipelineConfig", "QwenImageBundle", "QwenImageTextEmbedStage", "QwenImagePipeline", "PROMPT_PREFIX", "PROMPT_SUFFIX"]
