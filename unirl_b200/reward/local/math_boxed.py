"""Reference-compatible import path (``unirl.reward.local.math_boxed``); the scorer lives in ``rules.py``."""
from unirl_b200.reward.local.rules import MathBoxedRewardScorer, MathBoxedSpec, last_boxed, normalize_math, math_equal  # noqa: F401
