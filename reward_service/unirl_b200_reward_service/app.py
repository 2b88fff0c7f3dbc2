"""Reward service: FastAPI gateway in front of pools of scorer workers.

``POST /score``  ``{"scorers": [...], "weights": {...}, "items": [{"prompt", "image_png_b64" | "video_npy_b64" | "tokens", "metadata"}]}``
                 → ``{"rewards": [...], "component_rewards": {scorer: [...]}, "errors": [...]}`` (weighted sum of the scorers).
``GET /health``  liveness + loaded scorers;  ``GET /rewards`` the scorer catalogue.

Each scorer runs in its own worker pool (``ScorerPool``: N replicas, each pinned to a device, requests dispatched
round-robin through a thread pool so slow scorers do not block fast ones).  Parity: the external
``unirl-reward-service`` package (FastAPI + one actor pool per scorer; ``docs/ARCHITECTURE.md:18-90``).
"""

from __future__ import annotations

import itertools
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

import torch

from unirl_b200.reward.local.scorers import SCORERS, build_scorer
from unirl_b200.reward.remote import decode_image, decode_video
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.reward import RewardRequest


class ScorerPool:
    def __init__(self, name: str, replicas: int = 1, devices: Optional[List[str]] = None, **kw: Any):
        devices = devices or ["cpu"]
        self.name = name
        self.workers = [build_scorer(name, device=devices[i % len(devices)], **kw) if name not in ("geneval", "geneval2", "ocr") else build_scorer(name)
                        for i in range(max(1, replicas))]
        self.locks = [threading.Lock() for _ in self.workers]
        self._rr = itertools.cycle(range(len(self.workers)))
        self.calls, self.seconds = 0, 0.0

    def score(self, request: RewardRequest) -> List[float]:
        i = next(self._rr)
        t0 = time.perf_counter()
        with self.locks[i]:
            out = self.workers[i].compute_rewards(request)
        self.calls += 1
        self.seconds += time.perf_counter() - t0
        return [float(r) for r in out.rewards]


class RewardGateway:
    def __init__(self, scorers: Optional[Dict[str, Dict[str, Any]]] = None, max_parallel: int = 8):
        self.pools: Dict[str, ScorerPool] = {}
        self._cfg = scorers or {}
        self._lock = threading.Lock()
        self._ex = ThreadPoolExecutor(max_workers=max_parallel)

    def pool(self, name: str) -> ScorerPool:
        with self._lock:
            if name not in self.pools:
                if name not in SCORERS:
                    raise KeyError(f"unknown scorer {name!r}")
                self.pools[name] = ScorerPool(name, **self._cfg.get(name, {}))
            return self.pools[name]

    def score(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        items = payload.get("items") or []
        names = payload.get("scorers") or ["clip"]
        weights = payload.get("weights") or {}
        n = len(items)
        errors: List[Optional[str]] = [None] * n
        gen: Dict[str, Any] = {}
        try:
            if items and items[0].get("image_png_b64"):
                imgs = [decode_image(it["image_png_b64"]) for it in items]
                size = imgs[0].shape[-2:]
                gen["image"] = Images(pixels=torch.stack([im if im.shape[-2:] == size else torch.nn.functional.interpolate(im[None], size=size)[0] for im in imgs]))
            if items and items[0].get("video_npy_b64"):
                gen["video"] = [decode_video(it["video_npy_b64"]) for it in items]
            if items and items[0].get("tokens") is not None:
                gen["tokens"] = [torch.tensor(it["tokens"]) for it in items]
        except Exception as e:  # noqa: BLE001
            return {"rewards": [0.0] * n, "component_rewards": {}, "errors": [f"decode failed: {e}"] * n}
        req = RewardRequest(primitives={"text": Texts.from_list([it.get("prompt", "") for it in items])}, generated=gen,
                            metadata=[it.get("metadata") for it in items], sample_ids=[str(i) for i in range(n)])
        futures = {name: self._ex.submit(self.pool(name).score, req) for name in names}
        comps: Dict[str, List[float]] = {}
        for name, f in futures.items():
            try:
                comps[name] = f.result()
            except Exception as e:  # noqa: BLE001
                errors = [f"{name}: {e}"] * n
                comps[name] = [0.0] * n
        total = [sum(float(weights.get(k, 1.0)) * v[i] for k, v in comps.items()) for i in range(n)]
        return {"rewards": total, "component_rewards": comps, "errors": errors}

    def stats(self) -> Dict[str, Any]:
        return {k: {"replicas": len(p.workers), "calls": p.calls, "seconds": round(p.seconds, 3)} for k, p in self.pools.items()}


def create_app(scorers: Optional[Dict[str, Dict[str, Any]]] = None):
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="unirl_b200 reward service")
    gw = RewardGateway(scorers)
    app.state.gateway = gw

    @app.get("/health")
    def health() -> Dict[str, Any]:
        return {"status": "ok", "loaded": gw.stats()}

    @app.get("/rewards")
    def rewards() -> Dict[str, Any]:
        return {"scorers": sorted(SCORERS)}

    @app.post("/score")
    def score(payload: Dict[str, Any]) -> Dict[str, Any]:
        try:
            return gw.score(payload)
        except KeyError as e:
            raise HTTPException(status_code=404, detail=str(e)) from e

    return app


def main() -> None:
    import argparse

    import uvicorn

    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8077)
    ap.add_argument("--preload", default="", help="comma-separated scorers to load at start-up")
    a = ap.parse_args()
    app = create_app()
    for name in filter(None, a.preload.split(",")):
        app.state.gateway.pool(name)
    uvicorn.run(app, host=a.host, port=a.port)


if __name__ == "__main__":
    main()
