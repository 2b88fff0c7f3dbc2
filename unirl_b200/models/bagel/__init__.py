"""Bagel: unified mixture-of-transformers text-to-image model — every layer holds one parameter set for text /
understanding tokens and one for generated-image tokens (hard routing by modality), image generation by flow matching on
latent patch tokens.  Built on :mod:`unirl_b200.models.unified` with ``modality_experts=True``; the flow forward runs with
gradients enabled for training.  Parity: ``unirl/models/bagel/{bundle,diffusion,rl_ops}.py``."""
from dataclasses import dataclass

from unirl_b200.models.unified import UnifiedBundle, UnifiedConditions, UnifiedPipeline, UnifiedPipelineConfig


@dataclass
class BagelPipelineConfig(UnifiedPipelineConfig):
    pretrained_model_ckpt_path: str = "random:bagel-7b"


class BagelBundle(UnifiedBundle):
    pass


class BagelPipeline(UnifiedPipeline):
    @classmethod
    def from_config(cls, config: BagelPipelineConfig) -> "BagelPipeline":
        return cls(BagelBundle.from_config(config))


BagelConditions = UnifiedConditions

__all__ = ["BagelPipelineConfig", "BagelBundle", "BagelPipeline", "BagelConditions"]
