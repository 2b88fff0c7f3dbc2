"""Composed (AR → diffusion) rollout engine."""
from unirl_b200.rollout.engine.composed.engine import ComposedRolloutEngine, extract_enhanced_prompt

__all__ = ["ComposedRolloutEngine", "extract_enhanced_prompt"]
