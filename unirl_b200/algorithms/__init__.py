"""Loss nodes: GRPO / DRPO (token level), FlowGRPO / FlowDPPO / DiffusionNFT (flow matching).

DanceGRPO = FlowGRPO + ``DanceSDEStrategy``; MixGRPO = FlowGRPO + ``WindowScheduler`` (recipes, not classes).
"""
from unirl_b200.algorithms.base import AlgorithmStepResult, StageAlgorithm  # noqa: F401
from unirl_b200.algorithms.diffusionnft import DiffusionNFT  # noqa: F401
from unirl_b200.algorithms.drpo import DRPO  # noqa: F401
from unirl_b200.algorithms.flowdppo import FlowDPPO  # noqa: F401
from unirl_b200.algorithms.flowgrpo import FlowGRPO  # noqa: F401
from unirl_b200.algorithms.grpo import GRPO  # noqa: F401
