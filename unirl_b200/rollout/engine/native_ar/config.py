"""Config of the native AR rollout engine.

Field names follow the reference's SGLang LLM engine config (``unirl/rollout/engine/sglang_llm/config.py``)
where the concept carries over (``tp_size``, ``max_new_tokens``, sampling defaults, ``samples_pre_expanded``,
``engine_kwargs.mem_fraction_static`` / ``disable_cuda_graph`` / ``cuda_graph_max_bs``), so a recipe only swaps
the engine block.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional


@dataclass
class NativeAREngineConfig:
    pretrained_model_ckpt_path: str = "random:tiny"
    tokenizer_ckpt_path: Optional[str] = None
    model_precision: str = "bf16"
    tp_size: int = 1
    max_new_tokens: int = 512
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    page_size: int = 64
    max_running_requests: int = 256
    prefill_token_budget: int = 16384
    kv_cache_tokens: Optional[int] = None
    poll_interval: int = 64
    samples_pre_expanded: bool = True
    share_trainer_weights: bool = True  # colocated + tp_size==1: alias the trainer's bf16 replica (zero-copy sync)
    init_seed: int = 0
    seed: int = 0
    model_overrides: Dict[str, Any] = field(default_factory=dict)
    engine_kwargs: Dict[str, Any] = field(default_factory=dict)
    chat_template_kwargs: Dict[str, Any] = field(default_factory=dict)
    concurrency: int = 16  # accepted for recipe compatibility (no HTTP fan-out here)
    detokenize: bool = True
    tp_collectives: str = "fused"  # fused | nccl
    share_prefix: bool = True  # samples of one prompt share the prompt's KV pages; decode reads them once per group (cascade attention)

    @property
    def use_cuda_graph(self) -> bool:
        return not bool(self.engine_kwargs.get("disable_cuda_graph", False))


__all__ = ["NativeAREngineConfig"]
