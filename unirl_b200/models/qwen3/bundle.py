"""``Qwen3Bundle`` — the trainable transformer + tokenizer.

Loads a Hugging Face checkpoint directory (``config.json`` + ``*.safetensors``) into the native
fused-parameter module, or builds a random-init model from a preset (``random:tiny``,
``random:qwen3-4b``).  Parity: ``unirl/models/qwen3/bundle.py:37-99`` (which wraps ``AutoModelForCausalLM``).
"""

from __future__ import annotations

import glob
import json
import os
from typing import Any, Dict, Optional

import torch

from unirl_b200.models.qwen3.config import Qwen3PipelineConfig
from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.models.types import Bundle
from unirl_b200.utils.dtypes import parse_torch_dtype

PRESETS = {"tiny": Qwen3Config.tiny, "qwen3-4b": Qwen3Config.qwen3_4b, "qwen3_4b": Qwen3Config.qwen3_4b}


def resolve_model_config(path: str, overrides: Optional[Dict[str, Any]] = None) -> Qwen3Config:
    if path.startswith("random:"):
        cfg = PRESETS[path.split(":", 1)[1].lower()]()
    else:
        with open(os.path.join(path, "config.json")) as f:
            cfg = Qwen3Config.from_hf_dict(json.load(f))
    for k, v in (overrides or {}).items():
        setattr(cfg, k, v)
    return cfg


class Qwen3Bundle(Bundle):
    def __init__(self, transformer: Qwen3Transformer, tokenizer: Any, config: Qwen3PipelineConfig):
        super().__init__()
        self.transformer = transformer
        self.tokenizer = tokenizer
        self.config = config

    @property
    def model_config(self) -> Qwen3Config:
        return self.transformer.cfg

    @classmethod
    def from_config(cls, config: Qwen3PipelineConfig) -> "Qwen3Bundle":
        path = config.pretrained_model_ckpt_path
        mcfg = resolve_model_config(path, config.model_overrides)
        dtype = parse_torch_dtype(config.model_precision)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = Qwen3Transformer(mcfg, dtype=dtype, device=device, gradient_checkpointing=config.use_gradient_checkpointing)
        if path.startswith("random:"):
            model.init_weights(config.init_seed)
        else:
            from safetensors.torch import load_file

            sd: Dict[str, torch.Tensor] = {}
            for shard in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
                sd.update(load_file(shard))
            model.load_hf_state_dict(sd)
        tok = load_tokenizer(config.tokenizer_ckpt_path or (None if path.startswith("random:") else path), mcfg.vocab_size, config.trust_remote_code)
        return cls(model, tok, config)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


__all__ = ["Qwen3Bundle", "resolve_model_config"]
