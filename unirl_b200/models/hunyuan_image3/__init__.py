"""HunyuanImage-3: unified AR + DiT mixture-of-experts model (64 routed experts, 8 active, one shared), four request modes
``t2t / i2t / t2i / it2i`` on one shared transformer.  Built on :mod:`unirl_b200.models.unified`.
Parity: ``unirl/models/hunyuan_image3/`` (``from_meta_config`` + per-rank ``materialize``, fused multimodal condition)."""
from dataclasses import dataclass

from unirl_b200.models.unified import UnifiedBundle, UnifiedConditions, UnifiedPipeline, UnifiedPipelineConfig


@dataclass
class HunyuanImage3PipelineConfig(UnifiedPipelineConfig):
    pretrained_model_ckpt_path: str = "random:hunyuan-image3"
    recaption: bool = True


class HunyuanImage3Bundle(UnifiedBundle):
    """``from_meta_config`` builds the 80B mixture-of-experts tree without memory; ``materialize(device, with_aux, ep)`` allocates and fills
    this rank's share (its experts only under expert parallelism), from checkpoint shards or by name-keyed random init
    (:class:`unirl_b200.models.unified.pipeline.UnifiedBundle`)."""


class HunyuanImage3Pipeline(UnifiedPipeline):
    @classmethod
    def from_config(cls, config: HunyuanImage3PipelineConfig) -> "HunyuanImage3Pipeline":
        return cls(HunyuanImage3Bundle.from_config(config))


HunyuanImage3Conditions = HunyuanImage3ARConditions = HunyuanImage3DiffusionConditions = UnifiedConditions  # one record serves the text and the image track

__all__ = ["HunyuanImage3PipelineConfig", "HunyuanImage3Bundle", "HunyuanImage3Pipeline", "HunyuanImage3Conditions", "HunyuanImage3ARConditions",
           "HunyuanImage3DiffusionConditions"]
