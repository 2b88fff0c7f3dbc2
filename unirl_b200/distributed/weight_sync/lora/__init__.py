from unirl_b200.distributed.weight_sync.lora.base import LoraWeightSyncBase  # noqa: F401
from unirl_b200.distributed.weight_sync.lora.local import LocalLoraWeightSync  # noqa: F401
from unirl_b200.distributed.weight_sync.lora.remote import RemoteLoraWeightSync  # noqa: F401
