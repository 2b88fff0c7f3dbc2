from unirl_b200.distributed.group.comm import Comm  # noqa: F401
from unirl_b200.distributed.group.device_pool import DevicePool, WorkerDied, WorkerError, WorkerTimeout  # noqa: F401
from unirl_b200.distributed.group.dispatch import Dispatch, Execute, distributed  # noqa: F401
from unirl_b200.distributed.group.handle import Handle, HandleRef  # noqa: F401
from unirl_b200.distributed.group.placement import placement, remote, remote_cfg, remote_hydra  # noqa: F401
from unirl_b200.distributed.group.remote import RankInfo, Remote  # noqa: F401
from unirl_b200.distributed.group.worker import Worker  # noqa: F401
