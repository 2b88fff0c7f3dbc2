"""Reference-compatible import path (``unirl.reward.local.mathverify``); the scorer lives in ``rules.py``."""
from unirl_b200.reward.local.rules import MathVerifyRewardScorer, MathVerifySpec  # noqa: F401
