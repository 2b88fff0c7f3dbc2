"""``RemoteRewardBackend`` — HTTP client of the reward service (``POST /score``).

Images travel as base64 PNG (lossless), videos as base64 ``.npy`` uint8 frame stacks; requests are cut into batches of
``batch_size`` samples, up to ``concurrency`` batches in flight, each retried ``max_retries`` times with exponential
back-off.  A sample the service reports as failed makes the whole call fail (training on a silent zero reward is worse
than stopping).  Parity: ``unirl/reward/remote.py``.
"""

from __future__ import annotations

import base64
import io
import json
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from unirl_b200.reward.base import RewardBackend
from unirl_b200.types.reward import RewardRequest, RewardResponse


def encode_image(px: torch.Tensor) -> str:
    """``[3, H, W]`` in [0, 1] → base64 PNG."""
    from PIL import Image

    arr = (px.detach().float().clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def decode_image(b64: str) -> torch.Tensor:
    from PIL import Image

    arr = np.asarray(Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB"))
    return torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0


def encode_video(frames: torch.Tensor) -> str:
    buf = io.BytesIO()
    np.save(buf, (frames.detach().float().clamp(0, 1) * 255).round().to(torch.uint8).cpu().numpy())
    return base64.b64encode(buf.getvalue()).decode()


def decode_video(b64: str) -> torch.Tensor:
    return torch.from_numpy(np.load(io.BytesIO(base64.b64decode(b64)))).float() / 255.0


class RemoteRewardSpec:
    """Settings of the remote backend under the field names recipes written for the reference use (``config: {_target_: …RemoteRewardSpec,
    base_url, required_rewards, reward_weights, batch_size, timeout, max_retries, input_kind, …}``; ``unirl/reward/remote.py:625-653``)."""

    def __init__(self, base_url: str = "", required_rewards: Sequence[str] = (), reward_weights: Optional[Dict[str, float]] = None, batch_size: int = 8,
                 timeout: float = 300.0, max_retries: int = 3, retry_delay: float = 1.0, input_kind: str = "image", raise_on_failure: bool = True, **extra: Any):
        self.base_url, self.required_rewards, self.reward_weights = str(base_url), tuple(required_rewards), dict(reward_weights or {})
        self.batch_size, self.timeout, self.max_retries, self.retry_delay = int(batch_size), float(timeout), int(max_retries), float(retry_delay)
        self.input_kind, self.raise_on_failure, self.extra = str(input_kind), bool(raise_on_failure), dict(extra)


class RemoteRewardBackend(RewardBackend):
    def __init__(self, url: Optional[str] = None, scorers: Sequence[str] = ("clip",), weights: Optional[Dict[str, float]] = None, batch_size: int = 16, concurrency: int = 4,
                 max_retries: int = 5, timeout_s: float = 300.0, preferred_input_kind: str = "image", config: Optional[RemoteRewardSpec] = None, **_kw: Any):
        if config is not None:  # the spec form
            url = url or config.base_url
            scorers = tuple(config.required_rewards) or tuple(scorers)
            weights = config.reward_weights or weights
            batch_size, max_retries, timeout_s, preferred_input_kind = config.batch_size, config.max_retries, config.timeout, config.input_kind
        if not url:
            raise ValueError("RemoteRewardBackend needs the service's url (url=… or config.base_url)")
        self.url = url.rstrip("/")
        self.scorers, self.weights = list(scorers), dict(weights or {})
        self.batch_size, self.concurrency, self.max_retries, self.timeout_s = int(batch_size), int(concurrency), int(max_retries), float(timeout_s)
        self.preferred_input_kind = preferred_input_kind

    def _post(self, path: str, payload: Dict[str, Any]) -> Dict[str, Any]:
        data = json.dumps(payload).encode()
        delay = 0.5
        for attempt in range(self.max_retries + 1):
            try:
                req = urllib.request.Request(self.url + path, data=data, headers={"Content-Type": "application/json"})
                with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                    return json.loads(r.read())
            except (urllib.error.URLError, TimeoutError, ConnectionError) as e:
                if attempt == self.max_retries:
                    raise RuntimeError(f"reward service {self.url}{path} unreachable after {attempt + 1} attempts: {e}") from e
                time.sleep(delay)
                delay = min(delay * 2, 10.0)
        raise AssertionError("unreachable")

    def is_available(self) -> bool:
        try:
            req = urllib.request.Request(self.url + "/health")
            with urllib.request.urlopen(req, timeout=5.0) as r:
                return json.loads(r.read()).get("status") == "ok"
        except Exception:  # noqa: BLE001
            return False

    def _payloads(self, request: RewardRequest) -> List[Dict[str, Any]]:
        gen = request.generated
        n = request.batch_size
        texts = request.primitives.get("text")
        prompts = [t.to_str() for t in texts.to_list()] if hasattr(texts, "to_list") else [""] * n
        if len(prompts) != n and prompts and n % len(prompts) == 0:
            prompts = [p for p in prompts for _ in range(n // len(prompts))]
        meta = request.metadata or [None] * n
        items: List[Dict[str, Any]] = []
        img, vid = gen.get("image"), gen.get("video")
        px = getattr(img, "pixels", img) if img is not None else None
        clips = vid.to_list() if hasattr(vid, "to_list") else vid
        toks = gen.get("tokens")
        for i in range(n):
            it: Dict[str, Any] = {"prompt": prompts[i] if i < len(prompts) else "", "metadata": meta[i] if i < len(meta) else None}
            if px is not None:
                it["image_png_b64"] = encode_image(px[i])
            if clips is not None:
                it["video_npy_b64"] = encode_video(getattr(clips[i], "frames", clips[i]))
            if toks is not None:
                it["tokens"] = [int(x) for x in toks[i]]
            items.append(it)
        return [{"scorers": self.scorers, "weights": self.weights, "items": items[lo : lo + self.batch_size]} for lo in range(0, n, self.batch_size)]

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        batches = self._payloads(request)
        with ThreadPoolExecutor(max_workers=max(1, self.concurrency)) as ex:
            outs = list(ex.map(lambda p: self._post("/score", p), batches))
        rewards: List[float] = []
        comps: Dict[str, List[float]] = {}
        for o in outs:
            bad = [e for e in o.get("errors", []) if e]
            if bad:
                raise RuntimeError(f"reward service reported failures: {bad[:3]}")
            rewards += [float(r) for r in o["rewards"]]
            for k, v in (o.get("component_rewards") or {}).items():
                comps.setdefault(k, []).extend(float(x) for x in v)
        return RewardResponse.ok(rewards, comps, time.perf_counter() - t0)


__all__ = ["RemoteRewardSpec", "RemoteRewardBackend", "encode_image", "decode_image", "encode_video", "decode_video"]
