"""``DiTBundle`` — trainable DiT + frozen text towers + latent codec + tokenizers + schedule policy.

Built from ``random:<preset>`` (random-init weights of the named architecture) or from a native checkpoint directory.
Parity: ``unirl/models/sd3/bundle.py``, ``unirl/models/wan21/bundle.py`` (which wrap diffusers / transformers loaders).
"""

from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch

from unirl_b200.models.dit.config import DiTPipelineConfig, FamilySpec, resolve_family
from unirl_b200.models.dit.modeling import DiTTransformer
from unirl_b200.models.dit.text_encoder import TextEncoder
from unirl_b200.models.dit.vae import LatentVAE
from unirl_b200.models.dit.vae_wan import AutoencoderKLWan, is_wan_vae
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.models.types import Bundle
from unirl_b200.sde.runtime import FlowMatchSchedulePolicy
from unirl_b200.types.conditions.base import Modality
from unirl_b200.utils.dtypes import parse_torch_dtype


def _is_image_kl(vae_dir: str) -> bool:
    """True for the ``vae`` folder of an image checkpoint whose codec is the published 2-D KL auto-encoder (SD3 / SD3.5 / FLUX-style)."""
    import json

    with open(os.path.join(vae_dir, "config.json")) as f:
        d = json.load(f)
    return d.get("_class_name", "AutoencoderKL") == "AutoencoderKL" and "block_out_channels" in d


class DiTBundle(Bundle):
    def __init__(self, transformer: DiTTransformer, text_encoders: Any, vae: LatentVAE, tokenizers: Any, config: DiTPipelineConfig, spec: FamilySpec):
        super().__init__()
        self.transformer, self.text_encoders, self.vae, self.tokenizers = transformer, list(text_encoders), vae, list(tokenizers)
        self.config, self.spec = config, spec
        self.pretrained_path = None if config.pretrained_model_ckpt_path.startswith("random:") else config.pretrained_model_ckpt_path
        self.modality = Modality.VIDEO if spec.transformer.is_video else Modality.IMAGE
        self.concat_image_latents = False

    @property
    def model_config(self):
        return self.transformer.cfg

    def schedule_policy(self) -> FlowMatchSchedulePolicy:
        t = self.spec.transformer
        patch = t.patch_size[-1] * (2 if self.spec.packed_latents else 1)
        return FlowMatchSchedulePolicy(shift=float(self.config.shift if self.config.shift is not None else self.spec.shift),
                                       use_dynamic_shifting=self.spec.use_dynamic_shifting, vae_scale_factor=t.vae_scale_factor, patch_size=patch)

    @classmethod
    def from_config(cls, config: DiTPipelineConfig, sp: Optional[Any] = None) -> "DiTBundle":
        path = config.pretrained_model_ckpt_path
        spec = resolve_family(path, config.model_overrides)
        dtype = parse_torch_dtype(config.model_precision)
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = DiTTransformer(spec.transformer, dtype=dtype, device=device, gradient_checkpointing=config.use_gradient_checkpointing, sp=sp)
        if path.startswith("random:"):
            model.init_weights(config.init_seed)
        else:
            from safetensors.torch import load_file

            native = os.path.join(path, "transformer.safetensors")
            if os.path.exists(native):
                missing, unexpected = model.load_state_dict(load_file(native), strict=False)
                if missing or unexpected:
                    raise RuntimeError(f"checkpoint/key mismatch: missing {missing[:5]} unexpected {unexpected[:5]}")
            else:
                # a diffusers layout: <path>/transformer/diffusion_pytorch_model*.safetensors in the family's own key grammar
                import glob

                from unirl_b200.models.dit.hf_keys import load_diffusers_transformer

                shards = sorted(glob.glob(os.path.join(path, "transformer", "diffusion_pytorch_model*.safetensors")))
                if not shards:
                    raise FileNotFoundError(f"{path}: neither transformer.safetensors nor transformer/diffusion_pytorch_model*.safetensors")
                sd = {}
                for f in shards:
                    sd.update(load_file(f))
                load_diffusers_transformer(model, sd, spec.transformer.name, strict=True)
        encoders, toks = [], []
        for i, c in enumerate(spec.text_encoders):
            # diffusers layout: text_encoder, text_encoder_2, text_encoder_3 (+ tokenizer, tokenizer_2, ...) next to the transformer
            suffix = "" if i == 0 else f"_{i + 1}"
            enc_dir = None if path.startswith("random:") else os.path.join(path, "text_encoder" + suffix)
            if enc_dir and os.path.isdir(enc_dir) and c.kind in ("clip", "t5", "llm"):  # "llm": a Qwen / LLaMA decoder, loaded into the package's own
                from unirl_b200.models.dit.text_keys import load_hf_text_encoder

                enc, loaded_cfg = load_hf_text_encoder(enc_dir, dtype=dtype, device=device)
                loaded_cfg.max_length, loaded_cfg.penultimate = c.max_length, c.penultimate  # sequence length and layer choice are the family's
                spec.text_encoders[i] = loaded_cfg
                encoders.append(enc)
                toks.append(load_tokenizer(os.path.join(path, "tokenizer" + suffix), loaded_cfg.vocab_size, True))
            else:
                encoders.append(TextEncoder(c, dtype=dtype, device=device).init_weights(config.init_seed + 1 + i))
                toks.append(load_tokenizer(None, c.vocab_size, True))
        vae_dir = None if path.startswith("random:") else os.path.join(path, "vae")
        has_vae = bool(vae_dir) and os.path.exists(os.path.join(vae_dir, "config.json"))
        if has_vae and _is_image_kl(vae_dir):
            from unirl_b200.models.dit.vae_kl import AutoencoderKL

            vae = AutoencoderKL.from_hf(vae_dir, device=device)  # fp32, as the codec is used
        elif has_vae and is_wan_vae(vae_dir):
            vae = AutoencoderKLWan.from_hf(vae_dir, device=device)  # the causal 3-D codec of WAN 2.1 / 2.2-14B and Qwen-Image
        else:
            vae = LatentVAE(spec.vae, device=device).init_weights(config.init_seed + 7)
        return cls(model, encoders, vae, toks, config, spec)

    def trainable_modules(self) -> Dict[str, torch.nn.Module]:
        return {"transformer": self.transformer}


__all__ = ["DiTBundle"]
