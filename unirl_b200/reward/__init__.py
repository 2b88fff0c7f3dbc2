"""Rewards: backend ABC, worker-side ``RewardService``, local scorers, HTTP client for the external service."""
from unirl_b200.reward.base import MultiRewardBackend, RewardBackend  # noqa: F401
from unirl_b200.reward.service import RewardService  # noqa: F401
