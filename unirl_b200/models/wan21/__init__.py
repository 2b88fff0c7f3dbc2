"""WAN 2.1 video DiT (T2V and I2V) on the generic DiT core.  Parity: ``unirl/models/wan21/``."""
from unirl_b200.models.wan21.pipeline import Wan21Bundle, Wan21Pipeline, Wan21PipelineConfig

from unirl_b200.models.dit.conditions import DiTConditions as Wan21Conditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["Wan21Conditions", "Wan21Bundle", "Wan21Pipeline", "Wan21PipelineConfig"]
