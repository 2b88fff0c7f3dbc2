"""Data sources: a shuffled, resumable prompt stream → ``RolloutInputs``.

``MultimodalRLDataSource(args)`` reads ``args.run.data_path`` / ``eval_data_path`` / ``seed`` and
``args.algorithm.prompts_per_rollout`` like the reference (``unirl/data/data_source.py:123-361``); media refs are
loaded and validated on demand (``:26-120``).  ``DefaultDataSource`` serves an in-memory prompt list
(``:363-413``).  ``SyntheticTokenDataSource`` emits uniform-random token-id prompts (no tokenizer) for
random-weight runs.  Resume = the trainer re-draws ``step`` batches to fast-forward the stream; the
permutation of epoch ``e`` depends only on ``(seed, e)``.
"""

from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from unirl_b200.data.datasets import PromptDataset, load_dataset
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.media import MediaRef
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.prompts import RolloutInputs


def load_media(ref: MediaRef, size: Optional[int] = None) -> torch.Tensor:
    """Image file → ``[3, H, W]`` float in [0, 1]; raises with the path on failure."""
    if not ref.is_local:
        raise ValueError(f"remote media is not reachable from this box: {ref.uri}")
    if not os.path.exists(ref.path):
        raise FileNotFoundError(f"media file missing: {ref.path}")
    from PIL import Image

    img = Image.open(ref.path).convert("RGB")
    if size:
        img = img.resize((size, size))
    return torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float() / 255.0


class _Stream:
    def __init__(self, n: int, seed: int):
        self.n, self.seed, self.epoch, self.cursor = n, int(seed), 0, 0
        self.perm = self._perm()

    def _perm(self) -> np.ndarray:
        return np.random.default_rng([self.seed, self.epoch]).permutation(self.n)

    def draw(self, k: int) -> List[int]:
        out: List[int] = []
        while len(out) < k:
            if self.cursor >= self.n:
                self.epoch, self.cursor = self.epoch + 1, 0
                self.perm = self._perm()
            take = min(k - len(out), self.n - self.cursor)
            out += self.perm[self.cursor : self.cursor + take].tolist()
            self.cursor += take
        return out


class DefaultDataSource:
    def __init__(self, prompts: List[str], seed: int = 0, metadata: Optional[List[Optional[Dict[str, Any]]]] = None, shuffle: bool = True):
        self.dataset = PromptDataset([{"prompt": p, "metadata": (metadata[i] if metadata else None), "media": None} for i, p in enumerate(prompts)])
        self.eval_dataset = self.dataset
        self._stream = _Stream(len(self.dataset), seed) if shuffle else None
        self._cursor = 0
        self._draws = 0

    def _indices(self, k: int) -> List[int]:
        if self._stream is not None:
            return self._stream.draw(k)
        out = [(self._cursor + i) % len(self.dataset) for i in range(k)]
        self._cursor += k
        return out

    def _build(self, rows: List[Dict[str, Any]], tag: str) -> RolloutInputs:
        self._draws += 1
        gids = [f"{tag}{self._draws}:{i}" for i in range(len(rows))]
        prims: Dict[str, Any] = {"text": Texts(texts=[r["prompt"] for r in rows])}
        if any(r.get("media") for r in rows):
            size = getattr(self, "image_size", None)
            prims["image"] = Images(pixels=torch.stack([load_media(r["media"][0], size) for r in rows]))
        return RolloutInputs(primitives=prims, sample_ids=[f"prompt:{g}:sample:0" for g in gids], group_ids=gids,
                             metadata=[r.get("metadata") for r in rows])

    def get_samples(self, batch_size: int) -> RolloutInputs:
        return self._build([self.dataset[i] for i in self._indices(batch_size)], "r")

    def get_eval_samples(self, n: int) -> RolloutInputs:
        n = min(n, len(self.eval_dataset))
        return self._build([self.eval_dataset[i] for i in range(n)], "e")


class MultimodalRLDataSource(DefaultDataSource):
    def __init__(self, args: Any):
        run = args["run"] if isinstance(args, dict) else args.run
        get = (lambda o, k, d=None: o.get(k, d)) if isinstance(run, dict) or hasattr(run, "get") else (lambda o, k, d=None: getattr(o, k, d))
        self.dataset = load_dataset(str(get(run, "data_path")))
        ev = get(run, "eval_data_path")
        self.eval_dataset = load_dataset(str(ev)) if ev and str(ev) != str(get(run, "data_path")) else self.dataset
        self.image_size = get(run, "image_size")
        self._stream = _Stream(len(self.dataset), int(get(run, "seed", 0)))
        self._cursor = 0
        self._draws = 0
        algo = args.get("algorithm") if hasattr(args, "get") else getattr(args, "algorithm", None)
        self.prompts_per_rollout = int((algo or {}).get("prompts_per_rollout", 0)) if algo is not None else 0


class SyntheticImageQuestionDataSource(DefaultDataSource):
    """Question + seeded random image per prompt: a dataset-free source for vision-language recipes and tests."""

    def __init__(self, questions: List[str], image_size: Any = (28, 28), seed: int = 0, shuffle: bool = True):
        super().__init__(list(questions), seed=seed, shuffle=shuffle)
        self._img_hw = (int(image_size[0]), int(image_size[1]))
        self._img_seed = int(seed)

    def _build(self, rows: List[Dict[str, Any]], tag: str) -> RolloutInputs:
        out = super()._build(rows, tag)
        g = torch.Generator().manual_seed(self._img_seed * 7919 + self._draws)
        out.primitives["image"] = Images(pixels=torch.rand(len(rows), 3, *self._img_hw, generator=g))
        return out


class SyntheticTokenDataSource:
    """Prompts of uniform-random token ids with lengths uniform in ``[min_len, max_len]`` (deterministic in ``seed``).

    Prompts travel as ``request_conditions["prompt"]`` (right-padded ids + mask); ``primitives["text"]`` carries
    placeholders so reward/request plumbing that counts prompts keeps working.
    """

    def __init__(self, vocab_size: int = 4096, min_len: int = 32, max_len: int = 64, seed: int = 0, reserved_low_ids: int = 16,
                 suffix_token_ids: Optional[List[int]] = None):
        self.vocab_size, self.min_len, self.max_len, self.seed = int(vocab_size), int(min_len), int(max_len), int(seed)
        self.low = int(reserved_low_ids)
        self.suffix = list(suffix_token_ids or [])
        self._draws = 0

    def _draw(self, n: int, tag: str) -> RolloutInputs:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + self._draws)
        self._draws += 1
        lens = torch.randint(self.min_len, self.max_len + 1, (n,), generator=g)
        rows = [torch.randint(self.low, self.vocab_size, (int(l),), generator=g).tolist() + self.suffix for l in lens]
        width = max(len(r) for r in rows)
        ids = torch.zeros(n, width, dtype=torch.long)
        mask = torch.zeros(n, width, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : len(r)] = torch.tensor(r)
            mask[i, : len(r)] = 1
        gids = [f"{tag}{self._draws}:{i}" for i in range(n)]
        inputs = RolloutInputs(primitives={"text": Texts(texts=[""] * n)}, sample_ids=[f"prompt:{g_}:sample:0" for g_ in gids], group_ids=gids,
                               metadata=[None] * n)
        inputs.primitives["prompt_tokens"] = TextTokenCondition(input_ids=ids, attention_mask=mask)
        return inputs

    def get_samples(self, batch_size: int) -> RolloutInputs:
        return self._draw(batch_size, "r")

    def get_eval_samples(self, n: int) -> RolloutInputs:
        return self._draw(n, "e")


__all__ = ["SyntheticImageQuestionDataSource", "DefaultDataSource", "MultimodalRLDataSource", "SyntheticTokenDataSource", "load_media"]
