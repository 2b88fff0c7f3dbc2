"""Reference-compatible import path for the config helpers (``unirl.utils.hydra``)."""
from unirl_b200.config.instantiate import parse_cfg as parse_hydra_cfg  # noqa: F401
from unirl_b200.distributed.group.placement import remote_cfg as remote_hydra  # noqa: F401
