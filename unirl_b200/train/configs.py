"""Training-side config dataclasses.  Field names follow ``unirl/train/configs.py:7-82`` and
``unirl/train/backend/base.py:18-91`` so reference recipes load unchanged."""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict, Optional, Tuple


@dataclass
class LoraConfig:
    rank: int = 8
    alpha: int = 16
    target_modules: Tuple[str, ...] = ("q_proj", "k_proj", "v_proj", "o_proj")
    dropout: float = 0.0
    bias: str = "none"
    task_type: str = "FEATURE_EXTRACTION"


@dataclass
class EmaLoraConfig(LoraConfig):
    default_adapter: str = "default"
    shadow_adapter: str = "old"
    ema_decay: float = 0.001
    ema_decay_type: str = "constant"
    ema_flat_steps: int = 0
    ema_uprate: float = 0.001
    ema_uphold: float = 0.5
    timing: str = "rollout_end"


@dataclass
class EmaFullConfig:
    target_decay: float = 0.9999
    timing: str = "optimizer_step"
    shadow_prefix: str = "shadow_"


@dataclass
class FSDPConfig:
    param_dtype: str = "bf16"
    cpu_offload: bool = False
    mixed_precision: bool = True
    fsdp_mode: str = "full"  # full | hybrid (HSDP: shard inside groups of `hsdp_shard_size` ranks, replicate across them)
    hsdp_shard_size: int = 8
    reshard_after_forward: bool = False  # False: ZeRO-2, bf16 replica resident (default: HBM is plentiful); True: ZeRO-3, gather around each block
    activation_checkpointing: bool = False
    sp_size: int = 1  # Ulysses sequence-parallel degree inside one data-parallel replica (the role must be created with parallel={"sp": n})
    cp_size: int = 1  # context-parallel ranks of the autoregressive replay (each sequence cut over the group); place the role with train_parallel={sp: cp_size}
    checkpoint_layers: Optional[int] = None  # with activation_checkpointing: recompute only the first N blocks (None = every block)
    use_torch_compile: bool = False  # accepted for recipe compatibility; there is no tracing compiler here
    defer_grad_sync: bool = False
    forward_prefetch: bool = False
    master_dtype: Optional[str] = None
    root_wrap: bool = True
    collectives: str = "fused"  # fused (peer-memory kernels) | nccl (baseline)


@dataclass
class OptimizerConfig:
    learning_rate: float = 1e-6
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    weight_decay: float = 0.01


@dataclass
class LrSchedulerConfig:
    type: str = "constant"
    warmup_steps: int = 0
    total_steps: int = 1000


@dataclass
class TrainTopology:
    dp_size: Optional[int] = None
    dp_replicate_size: int = 1
    dp_shard_size: Optional[int] = None
    tp_size: int = 1
    pp_size: int = 1
    sp_size: int = 1
    ep_size: int = 1
    cp_size: int = 1
    actor_count: Optional[int] = 1

    def __post_init__(self) -> None:
        for name in ("dp_replicate_size", "tp_size", "pp_size", "sp_size", "ep_size", "cp_size"):
            if int(getattr(self, name)) < 1:
                raise ValueError(f"TrainTopology.{name} must be >= 1")

    def to_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in asdict(self).items() if v is not None}


__all__ = ["LoraConfig", "EmaLoraConfig", "EmaFullConfig", "FSDPConfig", "OptimizerConfig", "LrSchedulerConfig", "TrainTopology"]
