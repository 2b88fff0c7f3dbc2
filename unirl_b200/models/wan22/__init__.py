"""WAN 2.2: two expert transformers routed by the noise level.  Parity: ``unirl/models/wan22/``."""
from unirl_b200.models.wan22.pipeline import Wan22Bundle, Wan22Pipeline, Wan22PipelineConfig, WanDualTransformer

__all__ = ["Wan22Bundle", "Wan22Pipeline", "Wan22PipelineConfig", "WanDualTransformer"]
