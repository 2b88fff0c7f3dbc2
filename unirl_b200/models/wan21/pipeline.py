"""WAN 2.1 — text-to-video and image-to-video.

Latents are 5-D ``(C, (F−1)/4+1, H/8, W/8)``.  Image-to-video concatenates, along channels, a 4-channel first-frame
mask and the 16-channel encoded first frame to the noisy latents (36 input channels); the condition travels as an
``ImageLatentCondition`` holding those 20 channels.  Parity: ``unirl/models/wan21/diffusion.py:62-158, 317-334, 340-468``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Optional

import torch

from unirl_b200.models.dit.bundle import DiTBundle
from unirl_b200.models.dit.config import DiTPipelineConfig
from unirl_b200.models.dit.pipeline import DiTPipeline
from unirl_b200.models.dit.clip_vision import CLIPVisionConfig, CLIPVisionTower
from unirl_b200.types.conditions import ImageEmbedCondition, ImageLatentCondition


@dataclass
class Wan21PipelineConfig(DiTPipelineConfig):
    pretrained_model_ckpt_path: str = "random:wan21-14b"
    image_to_video: bool = False
    max_sequence_length: int = 512
    image_encoder_ckpt_path: Optional[str] = None  # image-to-video checkpoints: where the first frame's image encoder lives (None: beside the transformer)
    clip_vision: bool = True  # image-to-video: the transformer also reads an image encoder's tokens (WAN 2.1; the 2.2 checkpoints do not)

    def __post_init__(self) -> None:
        parent = getattr(super(), "__post_init__", None)
        if parent is not None:
            parent()
        if "i2v" in str(self.pretrained_model_ckpt_path).lower():  # the published image-to-video checkpoints say so in their name
            self.image_to_video = True


class Wan21Bundle(DiTBundle):
    @classmethod
    def from_config(cls, config: Wan21PipelineConfig, sp: Optional[Any] = None) -> "Wan21Bundle":
        if config.image_to_video and "in_channels" not in config.model_overrides:
            from dataclasses import replace

            from unirl_b200.models.dit.config import resolve_family

            base = resolve_family(config.pretrained_model_ckpt_path).transformer
            c = base.in_channels  # noisy + 4 mask + first-frame channels enter the patch embedding
            extra = {"in_channels": 2 * c + 4, "out_channels": c}
            if config.clip_vision and "image_dim" not in config.model_overrides:
                tiny = "tiny" in str(base.name)
                extra["image_dim"] = CLIPVisionConfig.tiny().hidden_size if tiny else CLIPVisionConfig().hidden_size
            config = replace(config, model_overrides={**config.model_overrides, **extra})
        b = super().from_config(config, sp)
        b.concat_image_latents = bool(config.image_to_video)
        b.image_encoder = cls._load_image_encoder(config, b) if (config.image_to_video and b.model_config.image_dim) else None
        return b

    @staticmethod
    def _load_image_encoder(config: Wan21PipelineConfig, b: "Wan21Bundle") -> CLIPVisionTower:
        """The checkpoint's ``image_encoder`` folder (or ``image_encoder_ckpt_path``); random weights for the ``random:`` presets."""
        path = str(config.pretrained_model_ckpt_path)
        device = next(b.transformer.parameters()).device
        folder = config.image_encoder_ckpt_path or (None if path.startswith("random:") else os.path.join(path, "image_encoder"))
        if folder and os.path.exists(os.path.join(folder, "config.json")):
            return CLIPVisionTower.from_hf(folder, dtype=torch.float32, device=device)
        c = CLIPVisionConfig.tiny() if b.model_config.image_dim == CLIPVisionConfig.tiny().hidden_size else CLIPVisionConfig(hidden_size=b.model_config.image_dim)
        return CLIPVisionTower(c, torch.float32, device).init_weights(config.init_seed + 11)

    def image_embed_condition(self, image: torch.Tensor) -> ImageEmbedCondition:
        """``image [B, 3, H, W]`` in [0, 1] → the image encoder's penultimate hidden states, all tokens valid
        (``unirl/models/wan21/clip_vision_encode.py:65-83``)."""
        e = self.image_encoder.encode(image)
        return ImageEmbedCondition(embeds=e, attn_mask=torch.ones(e.shape[:2], dtype=torch.long, device=e.device))

    def first_frame_condition(self, image: torch.Tensor, num_latent_frames: int) -> ImageLatentCondition:
        """``image [B, 3, H, W]`` in [0, 1] → ``[B, 20, F, h, w]``: mask (first latent frame = 1) ++ the codec's latents of the clip
        "this frame, then grey" (``unirl/models/wan21/image_encode.py:75-125``: the published codec is causal in time, so the grey frames
        encode to latents that depend on the first frame; a codec without a video encoder pads the encoded frame with zeros)."""
        if hasattr(self.vae, "encode_video"):
            t = (num_latent_frames - 1) * self.vae.cfg.temporal_factor + 1
            clip = torch.full((image.shape[0], 3, t, *image.shape[-2:]), 0.5, dtype=image.dtype, device=image.device)  # 0 on the codec's [-1, 1] scale
            clip[:, :, 0] = image
            lat = self.vae.encode_video(clip)
            b, c, _, h, w = lat.shape
        else:
            z = self.vae.encode(image)  # [B, 16, h, w]
            b, c, h, w = z.shape
            lat = torch.zeros(b, c, num_latent_frames, h, w, dtype=z.dtype, device=z.device)
            lat[:, :, 0] = z
        mask = torch.zeros(b, 4, num_latent_frames, h, w, dtype=lat.dtype, device=lat.device)
        mask[:, :, 0] = 1.0
        return ImageLatentCondition(latents=torch.cat([mask, lat], 1))


class Wan21Pipeline(DiTPipeline):
    @classmethod
    def from_config(cls, config: Wan21PipelineConfig) -> "Wan21Pipeline":
        return cls(Wan21Bundle.from_config(config))

    def _conditions(self, req: Any, d: Any):
        """Image-to-video: the request's condition images (``primitives["image"]``, one per sample) become the mask + first-frame latents
        the transformer reads beside the noisy latents (``unirl/models/wan21/pipeline.py`` runs its image-encode stage at this point)."""
        cond = super()._conditions(req, d)
        images = (req.primitives or {}).get("image")
        if self.bundle.concat_image_latents and cond.image is None and images is not None:
            px = images.pixels if hasattr(images, "pixels") else images
            px = px.to(next(self.bundle.vae.parameters()).device).float()
            if tuple(px.shape[-2:]) != (int(d.height), int(d.width)):
                px = torch.nn.functional.interpolate(px, size=(int(d.height), int(d.width)), mode="bicubic", align_corners=False).clamp(0, 1)
            cond.image = self.bundle.first_frame_condition(px, self.latent_shape(d)[1])
            if self.bundle.image_encoder is not None and cond.image_embed is None:
                cond.image_embed = self.bundle.image_embed_condition((images.pixels if hasattr(images, "pixels") else images).float())
        return cond

    def latent_shape(self, sampling: Any):
        shape = super().latent_shape(sampling)
        t = self.bundle.model_config
        return ((t.out_channels or t.in_channels), *shape[1:]) if self.bundle.concat_image_latents else shape


__all__ = ["Wan21PipelineConfig", "Wan21Bundle", "Wan21Pipeline"]
