"""Z-Image: single-stream DiT over the concatenated text + latent sequence.  Parity: ``unirl/models/z_image/``."""
from unirl_b200.models.z_image.pipeline import ZImageBundle, ZImagePipeline, ZImagePipelineConfig

__all__ = ["ZImageBundle", "ZImagePipeline", "ZImagePipelineConfig"]
