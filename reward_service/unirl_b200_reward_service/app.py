"""Reward service: FastAPI gateway in front of pools of scorer workers.

``POST /score``  ``{"scorers": [...], "weights": {...}, "items": [{"prompt", "image_png_b64" | "video_npy_b64" | "tokens", "metadata"}]}``
                 → ``{"rewards": [...], "component_rewards": {scorer: [...]}, "errors": [...]}`` (weighted sum of the scorers).
``GET /health``  liveness + loaded scorers;  ``GET /rewards`` the scorer catalogue.

``POST /score``  request form: ``{"requests": [{"prompt", media..., "rewards": [names], "metadata"}]}`` → per request
                 ``{"rewards": {name: value}, "errors": {name: text}}`` (bucketed per reward, one call per bucket).

Each reward runs in its own worker group (``workers.py``: N replicas, whole GPUs owned exclusively by one replica, replicas in the
gateway process or in spawned processes that see only their GPUs; round-robin dispatch through a thread pool so slow rewards do not
block fast ones; a dead worker process is restarted on the next request).  Configuration is YAML (``config.py``).  Parity: the external
``unirl-reward-service`` package (FastAPI + one actor pool per scorer; ``docs/ARCHITECTURE.md:18-90``).
"""

from __future__ import annotations

import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

import torch

from unirl_b200.reward.local.scorers import SCORERS
from unirl_b200.reward.remote import decode_image, decode_video
from unirl_b200_reward_service.config import RewardModelCfg, ServiceCfg, load_config
from unirl_b200_reward_service.workers import WorkerGroup, WorkerPool
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.reward import RewardRequest


def _decode_items(items: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Media of a list of items → the ``generated`` dict of a ``RewardRequest`` (images resized to the first one's size)."""
    gen: Dict[str, Any] = {}
    if items and items[0].get("image_png_b64"):
        imgs = [decode_image(it["image_png_b64"]) for it in items]
        size = imgs[0].shape[-2:]
        gen["image"] = Images(pixels=torch.stack([im if im.shape[-2:] == size else torch.nn.functional.interpolate(im[None], size=size)[0] for im in imgs]))
    if items and items[0].get("video_npy_b64"):
        gen["video"] = [decode_video(it["video_npy_b64"]) for it in items]
    if items and items[0].get("tokens") is not None:
        gen["tokens"] = [torch.tensor(it["tokens"]) for it in items]
    return gen


def _request_of(items: List[Dict[str, Any]], gen: Dict[str, Any]) -> RewardRequest:
    return RewardRequest(primitives={"text": Texts.from_list([it.get("prompt", "") for it in items])}, generated=gen,
                         metadata=[it.get("metadata") for it in items], sample_ids=[str(i) for i in range(len(items))])


class RewardGateway:
    """Bucket / dispatch / gather in front of a :class:`WorkerPool`.

    Two payload forms.  Batch form: every item gets every scorer of ``scorers``; the answer carries the weighted sum.  Request form
    (``{"requests": [{..., "rewards": [names]}]}``): each request names the rewards it needs; requests are bucketed per reward, every
    bucket goes to that reward's group as one call, and the answer is per request ``{"rewards": {name: value}, "errors": {name: text}}``.
    A reward that fails (unknown name, worker error, dead worker process) costs only its own entries."""

    def __init__(self, scorers: Optional[Dict[str, Dict[str, Any]]] = None, max_parallel: int = 8, config: Optional[ServiceCfg] = None):
        if config is None:
            config = ServiceCfg(rewards=[RewardModelCfg(name=k, kwargs=dict(v)) for k, v in (scorers or {}).items()], max_parallel=max_parallel)
            self._lazy = [r for r in config.rewards]  # legacy form: load on first use
            config = ServiceCfg(rewards=[], max_parallel=max_parallel, isolation=config.isolation, gpu_ids=config.gpu_ids)
        else:
            self._lazy = []
        self.pool_ = WorkerPool(config)
        self._ex = ThreadPoolExecutor(max_workers=config.max_parallel)
        self._lock = threading.Lock()

    def pool(self, name: str) -> WorkerGroup:
        with self._lock:
            for r in list(self._lazy):
                if r.name == name:
                    self._lazy.remove(r)
                    return self.pool_.add(r)
        return self.pool_.get(name)

    # ---- batch form ------------------------------------------------------------------------------------------
    def score(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        if "requests" in payload:
            return self.score_requests(payload)
        items = payload.get("items") or []
        names = payload.get("scorers") or ["clip"]
        weights = payload.get("weights") or {}
        n = len(items)
        errors: List[Optional[str]] = [None] * n
        try:
            gen = _decode_items(items)
        except Exception as e:  # noqa: BLE001
            return {"rewards": [0.0] * n, "component_rewards": {}, "errors": [f"decode failed: {e}"] * n}
        req = _request_of(items, gen)
        for name in names:  # an unknown scorer is the caller's mistake: 404, not a per-item error
            self.pool(name)
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

    # ---- request form ----------------------------------------------------------------------------------------
    def score_requests(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        reqs = payload.get("requests") or []
        results = [{"rewards": {}, "errors": {}} for _ in reqs]
        buckets: Dict[str, List[int]] = {}
        for i, r in enumerate(reqs):
            for name in r.get("rewards") or []:
                buckets.setdefault(name, []).append(i)

        def run(name: str, idx: List[int]) -> List[float]:
            items = [reqs[i] for i in idx]
            return self.pool(name).score(_request_of(items, _decode_items(items)))

        futures = {name: self._ex.submit(run, name, idx) for name, idx in buckets.items()}
        for name, f in futures.items():
            try:
                vals = f.result()
                for i, v in zip(buckets[name], vals):
                    results[i]["rewards"][name] = float(v)
            except Exception as e:  # noqa: BLE001
                for i in buckets[name]:
                    results[i]["errors"][name] = f"{type(e).__name__}: {e}"
        return {"results": results}

    def stats(self) -> Dict[str, Any]:
        return self.pool_.stats()

    def close(self) -> None:
        self.pool_.close()
        self._ex.shutdown(wait=False)


def create_app(scorers: Optional[Dict[str, Dict[str, Any]]] = None, config: Optional[ServiceCfg] = None):
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="unirl_b200 reward service")
    gw = RewardGateway(scorers, config=config)
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
    ap.add_argument("--config", default=None, help="YAML service configuration (rewards, replicas, GPUs per replica, isolation)")
    a = ap.parse_args()
    cfg = load_config(a.config) if a.config else None
    if cfg is not None:
        a.host, a.port = cfg.host, cfg.port
    app = create_app(config=cfg)
    for name in filter(None, a.preload.split(",")):
        app.state.gateway.pool(name)
    uvicorn.run(app, host=a.host, port=a.port)


if __name__ == "__main__":
    main()
