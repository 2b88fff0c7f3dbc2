"""unirl_b200 — B200-native RL post-training for autoregressive and flow-matching policies."""

__version__ = "0.1.0"
