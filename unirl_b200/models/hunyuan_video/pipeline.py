"""HunyuanVideo: 20 double + 40 single blocks, guidance embedding, LLM + CLIP text, on the generic DiT core.

What the family changes (``unirl/models/hunyuan_video/diffusion.py:34-36,121-134``, ``text_embed.py:30-45,80-100``):

* **guidance is an input, not a second pass**: the distilled model takes the guidance scale as an embedded scalar; there is no
  cond / uncond stacking and a negative prompt is ignored;
* **prompt template**: the LLM tower sees the prompt inside an instruction template; the hidden states of the template's prefix are
  cropped off, so the conditioning sequence starts at the user's text.  The prefix length is the number of tokens the prefix itself
  tokenises to (95 with the published tokenizer);
* the pooled conditioning is the CLIP tower's pooled vector.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.conditions import DiTConditions
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage
from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.dit.text_embed import TextEmbedStage
from unirl_b200.types.conditions import TextEmbedCondition
from unirl_b200.types.primitives import Texts

PROMPT_PREFIX = ("<|start_header_id|>system<|end_header_id|>\n\nDescribe the video by detailing the following aspects: 1. The main content and theme of the video."
                 "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects."
                 "3. Actions, events, behaviors temporal relationships, physical movement changes of the objects."
                 "4. background environment, light, style and atmosphere."
                 "5. camera angles, movements, and transitions used in the video:<|eot_id|>"
                 "<|start_header_id|>user<|end_header_id|>\n\n")
PROMPT_SUFFIX = "<|eot_id|>"


@dataclass
class HunyuanVideoPipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-video"
    use_prompt_template: bool = True


class HunyuanVideoBundle(DiTBundle):
    pass


class HunyuanVideoTextEmbedStage(TextEmbedStage):
    """LLM tower on the templated prompt with the template prefix cropped; CLIP tower on the bare prompt for the pooled vector."""

    def __init__(self, *a: Any, use_template: bool = True, **k: Any):
        super().__init__(*a, **k)
        self.use_template = bool(use_template)

    @torch.no_grad()
    def embed(self, texts: Any) -> TextEmbedCondition:
        strs: List[str] = [t.to_str() if hasattr(t, "to_str") else str(t) for t in (texts.to_list() if isinstance(texts, Texts) else texts)]
        if not self.use_template:
            return super().embed(strs)
        enc, tok = self.encoders[0], self.tokenizers[0]
        crop = len(tok.encode(PROMPT_PREFIX))
        c = enc.cfg
        dev = next(enc.parameters()).device
        ids, mask = self._tokenize(tok, [PROMPT_PREFIX + s + PROMPT_SUFFIX for s in strs], min(c.max_length, self.max_sequence_length) + crop, c.eos_token_id,
                                   c.vocab_size)
        seq, _ = enc(ids.to(dev), mask.to(dev))
        seq, mask = seq[:, crop:], mask[:, crop:].to(dev)
        pooled = self._encode_one(1, strs)[1] if len(self.encoders) > 1 else None
        if self.text_dim and seq.shape[-1] != self.text_dim:
            seq = torch.nn.functional.pad(seq, (0, self.text_dim - seq.shape[-1])) if seq.shape[-1] < self.text_dim else seq[..., : self.text_dim]
        return TextEmbedCondition(embeds=seq, pooled=pooled, attn_mask=mask)


class HunyuanVideoDiffusionStage(DiTDiffusionStage):
    def _branches(self, x: torch.Tensor, sigma: torch.Tensor, cond: DiTConditions, p: DiTDiffusionParams) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        model = self.bundle.transformer
        t = sigma.to(x.device).float().reshape(-1).expand(x.shape[0]) * 1000.0
        g = p.distilled_guidance_scale if p.distilled_guidance_scale is not None else p.guidance_scale
        guidance = torch.full((x.shape[0],), float(g) * 1000.0, device=x.device) if model.cfg.guidance_embed else None
        txt = cond.text
        return model(x, t, txt.embeds, txt.pooled, txt.attn_mask, guidance).float(), None  # one pass: the guidance scale is an input of the distilled model


class HunyuanVideoPipeline(DiTPipeline):
    def __init__(self, bundle, **options):
        super().__init__(bundle, **options)
        spec, cfg = bundle.spec, bundle.config
        self.diffusion = HunyuanVideoDiffusionStage(bundle, spec.default_strategy, cfg.autocast_precision)
        self.text_embed = HunyuanVideoTextEmbedStage(bundle.text_encoders, bundle.tokenizers, spec.text_combine, spec.transformer.text_dim, cfg.max_sequence_length,
                                                     use_template=bool(getattr(cfg, "use_prompt_template", True)))

    @classmethod
    def from_config(cls, config: HunyuanVideoPipelineConfig) -> "HunyuanVideoPipeline":
        return cls(HunyuanVideoBundle.from_config(config))


__all__ = ["HunyuanVideoPipelineConfig", "HunyuanVideoBundle", "HunyuanVideoTextEmbedStage", "HunyuanVideoDiffusionStage", "HunyuanVideoPipeline", "PROMPT_PREFIX"]
