"""dtype name parsing shared by configs.  Parity: ``unirl/utils/dtypes.py``."""

from __future__ import annotations

from typing import Any

import torch

_NAMES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16, "half": torch.float16,
          "fp32": torch.float32, "float32": torch.float32, "float": torch.float32, "fp64": torch.float64, "float64": torch.float64}


def parse_torch_dtype(value: Any) -> torch.dtype:
    if isinstance(value, torch.dtype):
        return value
    key = str(value).lower().replace("torch.", "")
    if key not in _NAMES:
        raise ValueError(f"unknown precision '{value}' (expected one of {sorted(_NAMES)})")
    return _NAMES[key]


def dtype_name(dtype: torch.dtype) -> str:
    return {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32", torch.float64: "fp64"}.get(dtype, str(dtype))


__all__ = ["parse_torch_dtype", "dtype_name"]
