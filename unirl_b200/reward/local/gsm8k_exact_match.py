"""Reference-compatible import path (``unirl.reward.local.gsm8k_exact_match``); the scorer lives in ``rules.py``."""
from unirl_b200.reward.local.rules import GSM8KExactMatchRewardScorer, GSM8KExactMatchSpec  # noqa: F401
