"""Reference-compatible import path (``unirl.reward.local.mc_exact_match``); the scorer lives in ``rules.py``."""
from unirl_b200.reward.local.rules import MCExactMatchRewardScorer, MCExactMatchSpec  # noqa: F401
