"""Construction config shared by every DiT-family pipeline, and the preset table of model geometries.

``pretrained_model_ckpt_path`` is either ``"random:<preset>"`` (random-init weights of the named architecture — the
form benchmarks and tests use) or a directory holding a native checkpoint (``transformer.safetensors`` in this
package's key grammar plus ``config.json``).  Field names follow ``unirl/models/sd3/config.py`` / ``wan21/config.py``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from unirl_b200.models.dit.modeling import DiTConfig
from unirl_b200.models.dit.text_encoder import TextEncoderConfig
from unirl_b200.models.dit.vae import VAEConfig


@dataclass
class DiTPipelineConfig:
    __extra_fields_ok__ = True  # recipes may carry fields of other loaders (config.instantiate.call_target keeps them as attributes)
    pretrained_model_ckpt_path: str = "random:tiny-sd3"
    model_precision: Any = "bf16"
    device: Any = None
    autocast_precision: str = "bf16"
    trajectory_precision: str = "fp32"
    logprob_precision: str = "fp32"
    use_gradient_checkpointing: bool = False
    shift: Optional[float] = None
    use_lora: bool = False
    lora_target_modules: Optional[List[str]] = None
    weight_sync_param_name_prefix: str = "transformer."
    lora_materialization: str = "merged_dense"
    max_sequence_length: int = 256
    negative_prompt: str = ""
    model_overrides: Dict[str, Any] = field(default_factory=dict)
    init_seed: int = 0
    decode_images: bool = True
    sp_size: int = 1  # Ulysses sequence-parallel degree inside one replica

    def __post_init__(self) -> None:
        from unirl_b200.utils.dtypes import parse_torch_dtype

        parse_torch_dtype(self.model_precision)


@dataclass
class FamilySpec:
    """Everything that distinguishes one model family: transformer geometry, text towers, codec, schedule defaults."""

    transformer: DiTConfig
    text_encoders: List[TextEncoderConfig]
    text_combine: str = "single"  # "single" | "sd3" (CLIP-L ++ CLIP-G channel-wise, padded, then T5 along the sequence)
    vae: VAEConfig = field(default_factory=VAEConfig)
    shift: float = 3.0
    use_dynamic_shifting: bool = False
    default_strategy: str = "cps"
    packed_latents: bool = False  # 2x2 latent patches folded into channels before the transformer (FLUX / Qwen-Image style)


def _tiny(name: str, **kw: Any) -> DiTConfig:
    base = dict(name=name, hidden_size=64, num_heads=4, head_dim=16, in_channels=4, text_dim=32, pooled_dim=32, num_joint_blocks=2, rope_axes=(4, 6, 6),
                pos_embed_max_size=32)
    base.update(kw)
    return DiTConfig(**base)


def _tiny_text(n: int = 1) -> List[TextEncoderConfig]:
    return [TextEncoderConfig.tiny("clip"), TextEncoderConfig.tiny("clip"), TextEncoderConfig.tiny("t5")][:n] if n > 1 else [TextEncoderConfig.tiny("t5")]


PRESETS: Dict[str, Callable[[], FamilySpec]] = {
    # ---- Stable Diffusion 3.5 Medium: 24 MMDiT blocks, 1536 wide, dual attention in the first 13, sin-cos table 384
    "sd35-medium": lambda: FamilySpec(
        DiTConfig(name="sd35-medium", hidden_size=1536, num_heads=24, head_dim=64, in_channels=16, num_joint_blocks=24, dual_attention_blocks=tuple(range(13)),
                  text_dim=4096, pooled_dim=2048, pos_embed="sincos2d", pos_embed_max_size=384, pos_embed_base_size=64, final_text_block=False),
        [TextEncoderConfig.clip_l(), TextEncoderConfig.clip_g(), TextEncoderConfig.t5_xxl()], "sd3", VAEConfig(), 3.0, False, "cps"),
    "tiny-sd3": lambda: FamilySpec(_tiny("tiny-sd3", pos_embed="sincos2d", dual_attention_blocks=(0,), final_text_block=False, pooled_dim=64), _tiny_text(3), "sd3",
                                   VAEConfig.tiny(), 3.0, False, "cps"),
    # ---- WAN 2.1: cross-attention video DiT (14B: 40 blocks x 5120, 1.3B: 30 x 1536), UMT5 text, 3-D rope
    "wan21-14b": lambda: FamilySpec(
        DiTConfig(name="wan21-14b", hidden_size=5120, num_heads=40, head_dim=128, in_channels=16, num_joint_blocks=0, num_cross_blocks=40, ffn_dim=13824, text_dim=4096,
                  pooled_dim=0, rope_axes=(44, 42, 42), is_video=True, qk_norm_scope="full", text_in_layers=2, final_modulation="table"),
        [TextEncoderConfig.umt5_xxl()], "single", VAEConfig(latent_channels=16, scaling_factor=1.0, shift_factor=0.0), 3.0, False, "dance"),
    "wan21-1.3b": lambda: FamilySpec(
        DiTConfig(name="wan21-1.3b", hidden_size=1536, num_heads=12, head_dim=128, in_channels=16, num_joint_blocks=0, num_cross_blocks=30, ffn_dim=8960, text_dim=4096,
                  pooled_dim=0, rope_axes=(44, 42, 42), is_video=True, qk_norm_scope="full", text_in_layers=2, final_modulation="table"),
        [TextEncoderConfig.umt5_xxl()], "single", VAEConfig(latent_channels=16, scaling_factor=1.0, shift_factor=0.0), 3.0, False, "dance"),
    "tiny-wan": lambda: FamilySpec(_tiny("tiny-wan", num_joint_blocks=0, num_cross_blocks=2, pooled_dim=0, is_video=True, qk_norm_scope="full", text_in_layers=2,
                                         final_modulation="table"), _tiny_text(), "single", VAEConfig.tiny(), 3.0,
                                   False, "dance"),
    # ---- Qwen-Image: 60 joint blocks x 3072, packed 2x2 latents (64 channels), LLM text tower, dynamic shift
    "qwen-image": lambda: FamilySpec(
        DiTConfig(name="qwen-image", hidden_size=3072, num_heads=24, head_dim=128, in_channels=64, patch_size=(1, 1, 1), num_joint_blocks=60, text_dim=3584, pooled_dim=0,
                  rope_axes=(16, 56, 56)),
        [TextEncoderConfig("llm", 151936, 3584, 28, 28, 18944, 1024, 0, False)], "single", VAEConfig(latent_channels=16), 3.0, True, "flow", True),
    "tiny-qwen-image": lambda: FamilySpec(_tiny("tiny-qwen-image", in_channels=16, patch_size=(1, 1, 1), pooled_dim=0), [TextEncoderConfig.tiny("llm")], "single",
                                          VAEConfig.tiny(), 3.0, True, "flow", True),
    # ---- FLUX.2 klein: 5 double + 20 single blocks x 3072, guidance-distilled, empirical-mu schedule
    "flux2-klein": lambda: FamilySpec(
        DiTConfig(name="flux2-klein", hidden_size=3072, num_heads=24, head_dim=128, in_channels=128, patch_size=(1, 1, 1), num_joint_blocks=5, num_single_blocks=20,
                  text_dim=7680, pooled_dim=0, rope_axes=(32, 48, 48), guidance_embed=False),
        [TextEncoderConfig("llm", 151936, 2560, 36, 32, 9728, 512, 0, False)], "single", VAEConfig(latent_channels=32), 3.0, True, "flow", True),
    "tiny-flux2": lambda: FamilySpec(_tiny("tiny-flux2", in_channels=16, patch_size=(1, 1, 1), num_joint_blocks=1, num_single_blocks=2, pooled_dim=0),
                                     [TextEncoderConfig.tiny("llm")], "single", VAEConfig.tiny(), 3.0, True, "flow", True),
    # ---- Z-Image: single-stream DiT, 30 blocks x 3840
    "z-image": lambda: FamilySpec(
        DiTConfig(name="z-image", hidden_size=3840, num_heads=30, head_dim=128, in_channels=64, patch_size=(1, 1, 1), num_joint_blocks=0, num_single_blocks=30,
                  text_dim=2560, pooled_dim=0, rope_axes=(32, 48, 48)),
        [TextEncoderConfig("llm", 151936, 2560, 36, 32, 9728, 512, 0, False)], "single", VAEConfig(latent_channels=16), 3.0, False, "flow", True),
    "tiny-z-image": lambda: FamilySpec(_tiny("tiny-z-image", in_channels=16, patch_size=(1, 1, 1), num_joint_blocks=0, num_single_blocks=2, pooled_dim=0),
                                       [TextEncoderConfig.tiny("llm")], "single", VAEConfig.tiny(), 3.0, False, "flow", True),
    # ---- HunyuanVideo: 20 double + 40 single x 3072, guidance embed; 1.5: 54 double blocks x 2048
    "hunyuan-video": lambda: FamilySpec(
        DiTConfig(name="hunyuan-video", hidden_size=3072, num_heads=24, head_dim=128, in_channels=16, num_joint_blocks=20, num_single_blocks=40, text_dim=4096,
                  pooled_dim=768, rope_axes=(16, 56, 56), guidance_embed=True, is_video=True),
        [TextEncoderConfig("llm", 128320, 4096, 32, 32, 14336, 256, 0, False), TextEncoderConfig.clip_l()], "llm+clip", VAEConfig(latent_channels=16), 7.0, False, "flow"),
    "hunyuan-video15": lambda: FamilySpec(
        DiTConfig(name="hunyuan-video15", hidden_size=2048, num_heads=16, head_dim=128, in_channels=65, out_channels=32, patch_size=(1, 1, 1), num_joint_blocks=54, text_dim=3584,
                  pooled_dim=0, rope_axes=(16, 56, 56), is_video=True),
        [TextEncoderConfig("llm", 151936, 3584, 28, 28, 18944, 1000, 0, False), TextEncoderConfig.byt5_small()], "llm+glyph", VAEConfig(latent_channels=32, channel_mult=(1, 2, 4, 4, 4)), 7.0, False, "flow"),
    "tiny-hunyuan-video15": lambda: FamilySpec(_tiny("tiny-hunyuan-video15", in_channels=9, out_channels=4, patch_size=(1, 1, 1), pooled_dim=0, is_video=True),
                                               [TextEncoderConfig.tiny("llm"), TextEncoderConfig.tiny("t5", hidden=16)], "llm+glyph", VAEConfig.tiny(), 7.0, False, "flow"),
    "tiny-hunyuan-video": lambda: FamilySpec(_tiny("tiny-hunyuan-video", num_joint_blocks=1, num_single_blocks=1, guidance_embed=True, is_video=True),
                                             [TextEncoderConfig.tiny("llm"), TextEncoderConfig.tiny("clip")], "llm+clip", VAEConfig.tiny(), 7.0, False, "flow"),
}


def resolve_family(path: str, overrides: Optional[Dict[str, Any]] = None) -> FamilySpec:
    if path.startswith("random:"):
        key = path.split(":", 1)[1].lower()
        if key not in PRESETS:
            raise KeyError(f"unknown DiT preset {key!r}; known: {sorted(PRESETS)}")
        spec = PRESETS[key]()
    else:
        import json
        import os

        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        spec = PRESETS[d["preset"]]()
        for k, v in (d.get("transformer") or {}).items():
            setattr(spec.transformer, k, v)
    for k, v in (overrides or {}).items():
        setattr(spec.transformer, k, v)
    spec.transformer.__post_init__()
    return spec


__all__ = ["DiTPipelineConfig", "FamilySpec", "PRESETS", "resolve_family"]
