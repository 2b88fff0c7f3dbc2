"""``SD3Bundle`` — MMDiT + CLIP-L + CLIP-G + T5 + 16-channel VAE (``unirl/models/sd3/bundle.py``).

``pretrained_model_ckpt_path`` may also be a diffusers-format directory (``transformer/diffusion_pytorch_model*.safetensors``):
its transformer weights are converted through :mod:`unirl_b200.models.sd3.hf_keys`.
"""
from __future__ import annotations

import glob
import os
from typing import Any, Optional

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.sd3.config import SD3PipelineConfig


class SD3Bundle(DiTBundle):
    @classmethod
    def from_config(cls, config: SD3PipelineConfig, sp: Optional[Any] = None) -> "SD3Bundle":
        path = config.pretrained_model_ckpt_path
        shards = sorted(glob.glob(os.path.join(path, "transformer", "*.safetensors"))) if not path.startswith("random:") else []
        if not shards:
            return super().from_config(config, sp)
        from dataclasses import replace

        from safetensors.torch import load_file

        from unirl_b200.models.sd3.hf_keys import from_diffusers

        b = super().from_config(replace(config, pretrained_model_ckpt_path="random:sd35-medium"), sp)
        sd = {}
        for s in shards:
            sd.update(load_file(s))
        t = b.transformer.cfg
        missing, unexpected = b.transformer.load_state_dict(from_diffusers(sd, t.num_joint_blocks, t.dual_attention_blocks), strict=False)
        if unexpected:
            raise RuntimeError(f"unexpected keys after conversion: {unexpected[:5]}")
        b.pretrained_path = path
        return b


__all__ = ["SD3Bundle"]
