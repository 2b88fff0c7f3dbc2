"""WAN 2.1 video DiT (T2V and I2V) on the generic DiT core.  Parity: ``unirl/models/wan21/``."""
from unirl_b200.models.wan21.pipeline import Wan21Bundle, Wan21Pipeline, Wan21PipelineConfig

__all__ = ["Wan21Bundle", "Wan21Pipeline", "Wan21PipelineConfig"]
