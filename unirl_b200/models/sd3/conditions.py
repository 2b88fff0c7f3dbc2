"""SD3 conditions: joint text embeddings ``[B, 77 + L_t5, 4096]`` + pooled ``[B, 2048]`` (+ negative pair under CFG)."""
from unirl_b200.models.dit.conditions import DiTConditions as SD3Conditions

__all__ = ["SD3Conditions"]
