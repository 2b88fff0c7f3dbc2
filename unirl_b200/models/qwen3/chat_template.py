"""Chat-template stage: ``Texts`` → right-padded token ids (``Qwen3ARConditions``).

Parity: ``unirl/models/qwen3/chat_template.py:29-89`` (system instruction, ``enable_thinking`` kwarg,
prompt-length clamp, right padding with an attention mask).
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch

from unirl_b200.models.qwen3.conditions import Qwen3ARConditions
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.primitives import Texts


def pad_right(rows: List[List[int]], pad_id: int) -> TextTokenCondition:
    width = max((len(r) for r in rows), default=0)
    ids = torch.full((len(rows), width), int(pad_id), dtype=torch.long)
    mask = torch.zeros((len(rows), width), dtype=torch.long)
    for i, r in enumerate(rows):
        ids[i, : len(r)] = torch.tensor(r, dtype=torch.long)
        mask[i, : len(r)] = 1
    return TextTokenCondition(input_ids=ids, attention_mask=mask)


class Qwen3ChatTemplateStage:
    def __init__(self, bundle: Any, system_instruction: Optional[str] = None, max_prompt_length: int = 2048, enable_thinking: bool = False):
        self.bundle, self.system_instruction = bundle, system_instruction
        self.max_prompt_length, self.enable_thinking = int(max_prompt_length), bool(enable_thinking)

    def embed(self, p: Texts) -> Qwen3ARConditions:
        tok = self.bundle.tokenizer
        rows: List[List[int]] = []
        for text in p.texts:
            msgs = ([{"role": "system", "content": self.system_instruction}] if self.system_instruction else []) + [{"role": "user", "content": text}]
            try:
                ids = tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=True, enable_thinking=self.enable_thinking)
            except TypeError:
                ids = tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=True)
            ids = list(ids["input_ids"] if isinstance(ids, dict) else ids)
            rows.append(ids[-self.max_prompt_length :])
        return Qwen3ARConditions(prompt=pad_right(rows, tok.pad_token_id or 0))


__all__ = ["Qwen3ChatTemplateStage", "pad_right"]
