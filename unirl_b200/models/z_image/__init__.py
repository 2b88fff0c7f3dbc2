"""Z-Image: single-stream DiT over the concatenated text + latent sequence.  Parity: ``unirl/models/z_image/``."""
from unirl_b200.models.z_image.pipeline import ZImageBundle, ZImagePipeline, ZImagePipelineConfig

from unirl_b200.models.dit.conditions import DiTConditions as ZImageConditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["ZImageConditions", "ZImageBundle", "ZImagePipeline", "ZImagePipelineConfig"]
