from unirl_b200.distributed.weight_sync.full.base import FullWeightSync  # noqa: F401
from unirl_b200.distributed.weight_sync.full.ipc import IPCWeightSync  # noqa: F401
from unirl_b200.distributed.weight_sync.full.nccl import NCCLWeightSync  # noqa: F401
from unirl_b200.distributed.weight_sync.full.reshard import ReshardWeightSync  # noqa: F401
from unirl_b200.distributed.weight_sync.full.tensor import TensorWeightSync  # noqa: F401
