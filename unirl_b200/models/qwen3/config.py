"""Construction config of the Qwen3 AR pipeline.  Parity: ``unirl/models/qwen3/config.py`` (same field names).

``pretrained_model_ckpt_path`` may point at a Hugging Face checkpoint directory (``config.json`` +
safetensors) or be a synthetic spec ``"random:<preset>"`` (``tiny`` | ``qwen3-4b``) for random-init runs.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class Qwen3PipelineConfig:
    __extra_fields_ok__ = True  # recipes may carry fields of other loaders (config.instantiate.call_target keeps them as attributes)
    pretrained_model_ckpt_path: str = "random:tiny"
    tokenizer_ckpt_path: Optional[str] = None
    trust_remote_code: bool = True
    model_precision: Any = "bf16"
    device: Any = None
    autocast_precision: str = "bf16"
    logprob_precision: str = "fp32"
    use_gradient_checkpointing: bool = False
    weight_sync_param_name_prefix: str = "transformer."
    lora_materialization: str = "merged_dense"
    use_lora: bool = False
    lora_target_modules: Optional[List[str]] = None
    system_instruction: Optional[str] = None
    enable_thinking: bool = False
    model_overrides: Dict[str, Any] = field(default_factory=dict)
    init_seed: int = 0
    max_prompt_length: int = 2048

    def __post_init__(self) -> None:
        from unirl_b200.utils.dtypes import parse_torch_dtype

        parse_torch_dtype(self.model_precision)


__all__ = ["Qwen3PipelineConfig"]
