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
    def materialize(self, device, with_aux=True):
        """Weights are created directly on the target device by ``from_config``; moving is all that is left to do."""
        self.transformer.to(device)
        if with_aux:
            self.vae.to(device)


class HunyuanImage3Pipeline(UnifiedPipeline):
    @classmethod
    def from_config(cls, config: HunyuanImage3PipelineConfig) -> "HunyuanImage3Pipeline":
        return cls(HunyuanImage3Bundle.from_config(config))


HunyuanImage3Conditions = UnifiedConditions

__all__ = ["HunyuanImage3PipelineConfig", "HunyuanImage3Bundle", "HunyuanImage3Pipeline", "HunyuanImage3Conditions"]
