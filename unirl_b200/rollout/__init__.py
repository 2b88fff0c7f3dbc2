"""Rollout: engines that turn a ``RolloutReq`` into a ``RolloutResp``."""
