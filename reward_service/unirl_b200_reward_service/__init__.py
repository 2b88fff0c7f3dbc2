"""Stand-alone reward scoring service (FastAPI gateway + per-reward worker groups)."""
from unirl_b200_reward_service.app import RewardGateway, create_app
from unirl_b200_reward_service.config import RewardModelCfg, ServiceCfg, load_config
from unirl_b200_reward_service.workers import WorkerGroup, WorkerPool

__all__ = ["RewardGateway", "create_app", "RewardModelCfg", "ServiceCfg", "load_config", "WorkerGroup", "WorkerPool"]
