"""Native in-process diffusion rollout engine."""
from unirl_b200.rollout.engine.native_diffusion.engine import GraphedVelocity, NativeDiffusionEngineConfig, NativeDiffusionRolloutEngine

__all__ = ["NativeDiffusionRolloutEngine", "NativeDiffusionEngineConfig", "GraphedVelocity"]
