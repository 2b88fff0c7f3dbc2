"""Tokenizer access: Hugging Face tokenizers when a checkpoint directory exists, otherwise a
deterministic byte-level stand-in so that synthetic-weight runs (tests, benchmarks) need no files."""

from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence


class ByteTokenizer:
    """UTF-8 bytes offset past a few special ids; vocab may be larger than 256+specials (ids above decode to '')."""

    def __init__(self, vocab_size: int = 4096):
        self.vocab_size = int(vocab_size)
        self.pad_token_id, self.bos_token_id, self.eos_token_id = 0, 1, 2
        self._offset = 3
        self.chat_template = None

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = [self._offset + b for b in text.encode("utf-8")]
        return ([self.bos_token_id] if add_special_tokens else []) + ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        raw = bytes(i - self._offset for i in ids if self._offset <= i < self._offset + 256)
        return raw.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages: List[Dict[str, str]], tokenize: bool = False, add_generation_prompt: bool = True, **_kw: Any):
        text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages) + ("<|assistant|>\n" if add_generation_prompt else "")
        return self.encode(text) if tokenize else text

    def __call__(self, texts: Sequence[str], **_kw: Any) -> Dict[str, List[List[int]]]:
        return {"input_ids": [self.encode(t) for t in texts]}

    def __len__(self) -> int:
        return self.vocab_size


def load_tokenizer(path: Optional[str], vocab_size: int = 4096, trust_remote_code: bool = True) -> Any:
    if path and os.path.isdir(path) and any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(path, trust_remote_code=trust_remote_code)
        if tok.pad_token_id is None:
            tok.pad_token = tok.eos_token
        return tok
    return ByteTokenizer(vocab_size)


__all__ = ["ByteTokenizer", "load_tokenizer"]
