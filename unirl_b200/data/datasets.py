"""Prompt datasets: plain text files, jsonl with metadata, parquet math sets, VLM image+question rows.

Each dataset yields ``{"prompt": str, "metadata": dict | None, "media": [MediaRef] | None}``.
Parity: ``unirl/data/datasets.py`` (text prompt files; jsonl with geneval/ocr metadata; parquet DAPO-17k / GSM8K;
VLM image + question).
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterator, List, Optional

from unirl_b200.types.media import MediaRef


class PromptDataset:
    def __init__(self, rows: List[Dict[str, Any]]):
        self.rows = rows

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return self.rows[i]


def _row(prompt: str, metadata: Optional[Dict[str, Any]] = None, media: Optional[List[MediaRef]] = None) -> Dict[str, Any]:
    return {"prompt": prompt, "metadata": metadata, "media": media}


def load_text_prompts(path: str) -> PromptDataset:
    with open(path) as f:
        return PromptDataset([_row(line.strip()) for line in f if line.strip()])


def load_jsonl(path: str, prompt_key: str = "prompt", image_key: Optional[str] = None) -> PromptDataset:
    rows = []
    base = os.path.dirname(os.path.abspath(path))
    with open(path) as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            prompt = d.get(prompt_key) or d.get("question") or d.get("text") or d.get("problem")
            if prompt is None:
                raise KeyError(f"{path}: row lacks '{prompt_key}' / question / text / problem")
            media = None
            resolve = lambda u: u if os.path.isabs(u) or "://" in u else os.path.join(base, u)  # noqa: E731  (relative to the jsonl's folder)
            img = d.get(image_key or "image") or d.get("images")
            if img:
                imgs = img if isinstance(img, list) else [img]
                media = [MediaRef(resolve(i), "image") for i in imgs]
            elif d.get("media_refs"):  # [{"modality": "image", "role": "condition", "uri": "images/7.png"}, ...]
                media = [MediaRef(resolve(str(m["uri"])), str(m.get("modality", "image"))) for m in d["media_refs"] if m.get("uri")]
            meta = {k: v for k, v in d.items() if k not in (prompt_key, "image", "images", "media_refs", "metadata")}
            if isinstance(d.get("metadata"), dict):  # a nested metadata record is the row's metadata; sibling keys (prompt_id, ...) ride along
                meta.update(d["metadata"])
            elif d.get("metadata") is not None:
                meta["metadata"] = d["metadata"]
            rows.append(_row(str(prompt), meta or None, media))
    return PromptDataset(rows)


def load_parquet(path: str, prompt_key: str = "prompt", answer_key: str = "answer") -> PromptDataset:
    import pyarrow.parquet as pq

    table = pq.read_table(path).to_pylist()
    rows = []
    for d in table:
        p = d.get(prompt_key)
        if isinstance(p, list):  # chat-format prompt column
            p = next((m.get("content") for m in reversed(p) if m.get("role") == "user"), None)
        ans = d.get(answer_key)
        if ans is None and isinstance(d.get("reward_model"), dict):
            ans = d["reward_model"].get("ground_truth")
        rows.append(_row(str(p), {"answer": ans, **{k: v for k, v in d.items() if k in ("data_source", "ability", "extra_info")}}))
    return PromptDataset(rows)


def load_dataset(path: str, **kw: Any) -> PromptDataset:
    if path.endswith(".jsonl") or path.endswith(".json"):
        return load_jsonl(path, **{k: v for k, v in kw.items() if k in ("prompt_key", "image_key")})
    if path.endswith(".parquet"):
        return load_parquet(path, **{k: v for k, v in kw.items() if k in ("prompt_key", "answer_key")})
    return load_text_prompts(path)


__all__ = ["PromptDataset", "load_dataset", "load_text_prompts", "load_jsonl", "load_parquet"]
