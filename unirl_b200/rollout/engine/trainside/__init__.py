from unirl_b200.rollout.engine.trainside.engine import TrainsideRolloutEngine  # noqa: F401
