"""``QwenVLBundle`` — native Qwen2.5-VL (decoder + vision tower) and tokenizer.  Parity: ``unirl/models/qwen_vl/bundle.py``."""

from __future__ import annotations

import glob
import json
import os
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
        random_init = path.startswith("random:")
        if random_init:
            mcfg = PRESETS[path.split(":", 1)[1].lower()]()
        else:
            with open(os.path.join(path, "config.json")) as f:
                mcfg = QwenVLConfig.from_hf_dict(json.load(f))
        for k, v in (config.model_overrides or {}).items():
            setattr(mcfg, k, v)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = QwenVLTransformer(mcfg, dtype=parse_torch_dtype(config.model_precision), device=device,
                                  gradient_checkpointing=config.use_gradient_checkpointing)
        if random_init:
            model.init_weights(config.init_seed)
        else:
            from safetensors.torch import load_file

            sd: Dict[str, torch.Tensor] = {}
            for shard in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
                sd.update(load_file(shard))
            model.load_hf_state_dict(sd)
        if getattr(config, "freeze_vision_tower", False):
            model.visual.requires_grad_(False)
        tok = load_tokenizer(config.tokenizer_ckpt_path or (None if random_init else path), mcfg.vocab_size, config.trust_remote_code)
        return cls(model, tok, config)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


__all__ = ["QwenVLBundle"]
