"""WAN 2.2: two expert transformers routed by the noise level.  Parity: ``unirl/models/wan22/``."""
from unirl_b200.models.wan22.pipeline import Wan22Bundle, Wan22Pipeline, Wan22PipelineConfig, WanDualTransformer

from unirl_b200.models.dit.conditions import DiTConditions as Wan22Conditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["Wan22Conditions", "Wan22Bundle", "Wan22Pipeline", "Wan22PipelineConfig", "WanDualTransformer"]
