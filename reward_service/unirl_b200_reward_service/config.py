"""Service configuration: YAML → typed dataclasses, validated before any worker starts.

```yaml
host: 127.0.0.1
port: 8077
isolation: process            # process: one spawned worker process per replica | thread: replicas inside the gateway process
rewards:
  - name: clip                # the name requests use
    scorer: clip              # catalogue entry (default: the name)
    num_replicas: 2
    num_gpus: 1               # whole GPUs per replica; a GPU belongs to exactly one replica
    kwargs: {model_id: /models/clip-vit-large-patch14}
  - name: ocr
    num_gpus: 0               # CPU scorer
```
Parity: ``unirl-reward-service`` ``reward_service/config.py`` (``ServiceCfg`` / ``RewardModelCfg``; ``num_replicas >= 1``, ``num_gpus >= 0``, unique names).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class RewardModelCfg:
    name: str
    scorer: Optional[str] = None
    num_replicas: int = 1
    num_gpus: int = 0
    kwargs: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.scorer = self.scorer or self.name
        self.num_replicas, self.num_gpus = int(self.num_replicas), int(self.num_gpus)
        if self.num_replicas < 1:
            raise ValueError(f"reward {self.name!r}: num_replicas must be >= 1 (got {self.num_replicas})")
        if self.num_gpus < 0:
            raise ValueError(f"reward {self.name!r}: num_gpus must be >= 0 (got {self.num_gpus})")


@dataclass
class ServiceCfg:
    rewards: List[RewardModelCfg] = field(default_factory=list)
    host: str = "127.0.0.1"
    port: int = 8077
    isolation: str = "thread"
    gpu_ids: Optional[List[int]] = None  # GPUs the service may hand out (default: all visible ones)
    max_parallel: int = 8

    def __post_init__(self) -> None:
        if self.isolation not in ("thread", "process"):
            raise ValueError(f"isolation must be 'thread' or 'process' (got {self.isolation!r})")
        names = [r.name for r in self.rewards]
        dup = sorted({n for n in names if names.count(n) > 1})
        if dup:
            raise ValueError(f"duplicate reward names: {dup}")

    def gpus_needed(self) -> int:
        return sum(r.num_replicas * r.num_gpus for r in self.rewards)


def from_dict(d: Dict[str, Any]) -> ServiceCfg:
    rewards = [RewardModelCfg(**r) if isinstance(r, dict) else RewardModelCfg(name=str(r)) for r in (d.get("rewards") or [])]
    return ServiceCfg(rewards=rewards, **{k: v for k, v in d.items() if k != "rewards"})


def load_config(path: str) -> ServiceCfg:
    import yaml

    with open(path) as f:
        return from_dict(yaml.safe_load(f) or {})


__all__ = ["RewardModelCfg", "ServiceCfg", "from_dict", "load_config"]
