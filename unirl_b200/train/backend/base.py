"""Backend-agnostic training config re-exports (reference path ``unirl.train.backend.base``)."""
from unirl_b200.train.configs import LrSchedulerConfig, OptimizerConfig, TrainTopology  # noqa: F401
