from unirl_b200.train.backend.fsdp import FSDPBackend  # noqa: F401
