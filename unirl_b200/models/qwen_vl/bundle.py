"""``QwenVLBundle`` — native Qwen2.5-VL (decoder + vision tower) and tokenizer.  Parity: ``unirl/models/qwen_vl/bundle.py``."""

from __future__ import annotations

from typing import Any, Dict

import torch

from unirl_b200.models.qwen_vl.config import QwenVLPipelineConfig
from unirl_b200.models.qwen_vl.modeling import QwenVLConfig, QwenVLTransformer
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.models.types import Bundle
from unirl_b200.utils.dtypes import parse_torch_dtype

PRESETS = {"tiny-vl": QwenVLConfig.tiny, "qwen2.5-vl-7b": QwenVLConfig.qwen25_vl_7b}


class QwenVLBundle(Bundle):
    def __init__(self, transformer: QwenVLTransformer, tokenizer: Any, config: QwenVLPipelineConfig):
        super().__init__()
        self.transformer, self.tokenizer, self.config = transformer, tokenizer, config

    @property
    def model_config(self) -> QwenVLConfig:
        return self.transformer.cfg

    @classmethod
    def from_config(cls, config: QwenVLPipelineConfig) -> "QwenVLBundle":
        path = config.pretrained_model_ckpt_path
        if not path.startswith("random:"):
            raise NotImplementedError("QwenVLBundle loads random-init presets (random:tiny-vl, random:qwen2.5-vl-7b); HF checkpoint import is not wired yet")
        mcfg = PRESETS[path.split(":", 1)[1].lower()]()
        for k, v in (config.model_overrides or {}).items():
            setattr(mcfg, k, v)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = QwenVLTransformer(mcfg, dtype=parse_torch_dtype(config.model_precision), device=device,
                                  gradient_checkpointing=config.use_gradient_checkpointing).init_weights(config.init_seed)
        return cls(model, load_tokenizer(config.tokenizer_ckpt_path, mcfg.vocab_size, config.trust_remote_code), config)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


__all__ = ["QwenVLBundle"]
