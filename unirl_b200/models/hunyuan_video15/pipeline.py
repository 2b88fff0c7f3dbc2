"""HunyuanVideo 1.5: 54 joint blocks, 32-channel latents, on the generic DiT core.

What the family changes (``unirl/models/hunyuan_video15/diffusion.py:37,137-164,46``):

* **channel packing of the transformer input**: ``cat([latents, cond_latents, cond_mask], dim=1)`` -- the conditioning frame latents and a
  one-channel mask ride along with the noisy latents (32 + 32 + 1 = 65 input channels, 32 output channels).  Text-to-video has no
  conditioning frame: both extras are zeros; image-to-video puts the encoded first frame and a mask of ones at frame 0;
* true classifier-free guidance (two branches, ``uncond + g·(cond − uncond)``, no norm correction) whenever ``guidance_scale > 1``;
* **two text streams** (``unirl/models/hunyuan_video15/text_embed.py:42-210``): the prompt in a chat template with a fixed system
  message through the multimodal LLM's language model, the template's prefix cut from the hidden states (108 tokens with the published
  tokenizer); and a glyph stream: the quoted snippets of the prompt (straight or curly quotes, duplicates dropped), rewritten as
  ``Text "…". `` and run through a byte-level T5 encoder, all zeros with an all-zero mask for a prompt without quotes.  The transformer
  of this package takes one conditioning sequence, so the glyph tokens are zero-padded to the LLM width and appended along the token
  axis with their mask.  The language model's last hidden states are used (the reference reads the third from last).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.nn.functional as F

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.dit.text_embed import glyph_text
from unirl_b200.models.qwen_image.pipeline import QwenImageTextEmbedStage
from unirl_b200.types.conditions import TextEmbedCondition
from unirl_b200.types.primitives import Texts

SYSTEM_MESSAGE = ("You are a helpful assistant. Describe the video by detailing the following aspects: "
                  "1. The main content and theme of the video. "
                  "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects. "
                  "3. Actions, events, behaviors temporal relationships, physical movement changes of the objects. "
                  "4. background environment, light, style and atmosphere. "
                  "5. camera angles, movements, and transitions used in the video.")


@dataclass
class HunyuanVideo15PipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-video15"
    use_prompt_template: bool = True
    byt5_max_length: int = 256  # token cap of the glyph stream (quoted snippets only)


class HunyuanVideo15Bundle(DiTBundle):
    pass


class HunyuanVideo15DiffusionStage(DiTDiffusionStage):
    def _model_input(self, x: torch.Tensor, cond: DiTConditions) -> torch.Tensor:
        b, _, f, h, w = x.shape
        cond_latents = torch.zeros_like(x)
        cond_mask = torch.zeros(b, 1, f, h, w, dtype=x.dtype, device=x.device)
        img = None if cond.image is None else cond.image.latents
        if img is not None:  # image-to-video: the clean first frame and a mask that marks it
            img = img.to(x)
            img = img if img.dim() == 5 else img.unsqueeze(2)
            cond_latents[:, :, :1] = img[:, :, :1]
            cond_mask[:, :, :1] = 1
        return torch.cat([x, cond_latents, cond_mask], 1)


class HunyuanVideo15TextEmbedStage(QwenImageTextEmbedStage):
    """LLM stream in the family's chat template ++ glyph stream (second encoder, when the bundle has one)."""

    prefix = "<|im_start|>system\n" + SYSTEM_MESSAGE + "<|im_end|>\n<|im_start|>user\n"
    suffix = "<|im_end|>\n<|im_start|>assistant\n"
    token_cap = 1000

    @torch.no_grad()
    def embed(self, texts: Any) -> TextEmbedCondition:
        strs: List[str] = [t.to_str() if hasattr(t, "to_str") else str(t) for t in (texts.to_list() if isinstance(texts, Texts) else texts)]
        keep, self.combine = self.combine, "single"  # the LLM stream is the one-encoder path of the parent
        try:
            cond = super().embed(strs)
        finally:
            self.combine = keep
        if len(self.encoders) < 2:
            return cond
        seq, mask = self.append_glyph_stream(strs, cond.embeds, cond.attn_mask)
        return TextEmbedCondition(embeds=seq, pooled=None, attn_mask=mask)


class HunyuanVideo15Pipeline(DiTPipeline):
    def __init__(self, bundle, **options):
        super().__init__(bundle, **options)
        spec, cfg = bundle.spec, bundle.config
        self.diffusion = HunyuanVideo15DiffusionStage(bundle, spec.default_strategy, cfg.autocast_precision)
        self.text_embed = HunyuanVideo15TextEmbedStage(bundle.text_encoders, bundle.tokenizers, spec.text_combine, spec.transformer.text_dim,
                                                       min(int(cfg.max_sequence_length), HunyuanVideo15TextEmbedStage.token_cap),
                                                       use_template=bool(getattr(cfg, "use_prompt_template", True)),
                                                       glyph_max_length=int(getattr(cfg, "byt5_max_length", 256)))

    @classmethod
    def from_config(cls, config: HunyuanVideo15PipelineConfig) -> "HunyuanVideo15Pipeline":
        return cls(HunyuanVideo15Bundle.from_config(config))


__all__ = ["HunyuanVideo15PipelineConfig", "HunyuanVideo15Bundle", "HunyuanVideo15DiffusionStage", "HunyuanVideo15TextEmbedStage", "HunyuanVideo15Pipeline", "glyph_text"]
