"""Reward service sub-project: FastAPI gateway + scorer pools (see ``app.py``)."""
from unirl_b200_reward_service.app import RewardGateway, ScorerPool, create_app

__all__ = ["RewardGateway", "ScorerPool", "create_app"]
