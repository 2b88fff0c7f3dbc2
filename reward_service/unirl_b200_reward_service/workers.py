"""Worker pool of the reward service: one group of replicas per reward, whole GPUs owned exclusively by one replica.

``WorkerPool``   registry of groups + the GPU ledger (a GPU index is handed to exactly one replica; asking for more than there are fails
                 at start-up, before anything is loaded).
``WorkerGroup``  N replicas of one scorer, dispatched round-robin; a replica serves one request at a time.
``ThreadActor``  the scorer lives in the gateway process (cheap; CPU scorers, tests).
``ProcessActor`` the scorer lives in a spawned process that sees only its own GPUs (``CUDA_VISIBLE_DEVICES``): a scorer that
                 crashes or leaks takes its process with it, not the gateway; the group restarts the replica on the next request.
Parity: ``unirl-reward-service`` ``reward_service/workers/{pool,group,actor}.py`` (Ray actors there; spawned processes and pipes here).
"""

from __future__ import annotations

import itertools
import multiprocessing as mp
import os
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

from unirl_b200_reward_service.config import RewardModelCfg, ServiceCfg


def _build(scorer: str, gpus: Sequence[int], kwargs: Dict[str, Any], remapped: bool):
    from unirl_b200.reward.local.scorers import build_scorer

    kw = dict(kwargs)
    if scorer not in ("geneval", "geneval2", "ocr"):
        kw.setdefault("device", (f"cuda:{0 if remapped else gpus[0]}") if gpus else "cpu")
    return build_scorer(scorer, **kw)


class ThreadActor:
    def __init__(self, cfg: RewardModelCfg, gpus: Sequence[int]):
        self.cfg, self.gpus = cfg, list(gpus)
        self.scorer = _build(cfg.scorer, self.gpus, cfg.kwargs, remapped=False)
        self.lock = threading.Lock()

    def score(self, request: Any) -> List[float]:
        with self.lock:
            return [float(r) for r in self.scorer.compute_rewards(request).rewards]

    def close(self) -> None:
        self.scorer = None


def _process_main(conn: Any, scorer: str, gpus: List[int], kwargs: Dict[str, Any]) -> None:
    if gpus:
        os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in gpus)  # before the first CUDA call of this process
    try:
        s = _build(scorer, gpus, kwargs, remapped=True)
        conn.send(("ready", None))
    except Exception as e:  # noqa: BLE001
        conn.send(("failed", f"{type(e).__name__}: {e}"))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            return
        if msg is None:
            return
        try:
            conn.send(("ok", [float(r) for r in s.compute_rewards(msg).rewards]))
        except Exception as e:  # noqa: BLE001
            conn.send(("error", f"{type(e).__name__}: {e}"))


class ProcessActor:
    def __init__(self, cfg: RewardModelCfg, gpus: Sequence[int], start_timeout: float = 600.0):
        self.cfg, self.gpus, self.start_timeout = cfg, list(gpus), start_timeout
        self.lock = threading.Lock()
        self.proc: Optional[mp.Process] = None
        self.conn: Any = None
        self._start()

    def _start(self) -> None:
        ctx = mp.get_context("spawn")
        self.conn, child = ctx.Pipe()
        self.proc = ctx.Process(target=_process_main, args=(child, self.cfg.scorer, self.gpus, self.cfg.kwargs), daemon=True)
        self.proc.start()
        child.close()
        if not self.conn.poll(self.start_timeout):
            self.close()
            raise TimeoutError(f"reward {self.cfg.name!r}: worker did not come up within {self.start_timeout:.0f} s")
        kind, detail = self.conn.recv()
        if kind != "ready":
            self.close()
            raise RuntimeError(f"reward {self.cfg.name!r}: worker failed to load: {detail}")

    def score(self, request: Any, timeout: float = 600.0) -> List[float]:
        with self.lock:
            if self.proc is None or not self.proc.is_alive():
                self._start()  # the previous request killed the replica: bring a fresh one up
            try:
                self.conn.send(request)
                if not self.conn.poll(timeout):
                    raise TimeoutError(f"reward {self.cfg.name!r}: no answer within {timeout:.0f} s")
                kind, payload = self.conn.recv()
            except (EOFError, BrokenPipeError, ConnectionResetError) as e:
                self.close()
                raise RuntimeError(f"reward {self.cfg.name!r}: worker process died ({type(e).__name__})") from e
            if kind != "ok":
                raise RuntimeError(str(payload))
            return payload

    def close(self) -> None:
        try:
            if self.conn is not None:
                try:
                    self.conn.send(None)
                except Exception:  # noqa: BLE001
                    pass
                self.conn.close()
        finally:
            if self.proc is not None:
                self.proc.join(timeout=5)
                if self.proc.is_alive():
                    self.proc.kill()
            self.proc = self.conn = None


class WorkerGroup:
    def __init__(self, cfg: RewardModelCfg, gpu_sets: List[List[int]], isolation: str):
        cls = ProcessActor if isolation == "process" else ThreadActor
        self.cfg = cfg
        self.actors = [cls(cfg, g) for g in gpu_sets]
        self._rr = itertools.cycle(range(len(self.actors)))
        self._rr_lock = threading.Lock()
        self.calls, self.errors, self.seconds = 0, 0, 0.0

    def score(self, request: Any) -> List[float]:
        with self._rr_lock:
            i = next(self._rr)
        t0 = time.perf_counter()
        try:
            return self.actors[i].score(request)
        except Exception:
            self.errors += 1
            raise
        finally:
            self.calls += 1
            self.seconds += time.perf_counter() - t0

    def close(self) -> None:
        for a in self.actors:
            a.close()


class WorkerPool:
    def __init__(self, cfg: ServiceCfg):
        self.cfg = cfg
        self._free = list(cfg.gpu_ids) if cfg.gpu_ids is not None else self._visible_gpus()
        if cfg.gpus_needed() > len(self._free):
            raise ValueError(f"the configured rewards need {cfg.gpus_needed()} GPUs, the service may hand out {len(self._free)}")
        self.groups: Dict[str, WorkerGroup] = {}
        self.owned: Dict[str, List[List[int]]] = {}
        self._lock = threading.Lock()
        for r in cfg.rewards:
            self.add(r)

    @staticmethod
    def _visible_gpus() -> List[int]:
        try:
            import torch

            return list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
        except Exception:  # noqa: BLE001
            return []

    def add(self, r: RewardModelCfg) -> WorkerGroup:
        with self._lock:
            if r.name in self.groups:
                raise ValueError(f"reward {r.name!r} is already loaded")
            need = r.num_replicas * r.num_gpus
            if need > len(self._free):
                raise ValueError(f"reward {r.name!r} needs {need} GPUs, {len(self._free)} are free")
            sets = [[self._free.pop(0) for _ in range(r.num_gpus)] for _ in range(r.num_replicas)]
            try:
                g = WorkerGroup(r, sets, self.cfg.isolation)
            except Exception:
                self._free = [x for s in sets for x in s] + self._free
                raise
            self.groups[r.name], self.owned[r.name] = g, sets
            return g

    def get(self, name: str, autoload: bool = True) -> WorkerGroup:
        g = self.groups.get(name)
        if g is not None:
            return g
        from unirl_b200.reward.local.scorers import SCORERS

        if not autoload or name not in SCORERS:
            raise KeyError(f"unknown reward {name!r}")
        return self.add(RewardModelCfg(name=name))  # a catalogue scorer nobody configured: one CPU / default-device replica on first use

    def stats(self) -> Dict[str, Any]:
        return {k: {"replicas": len(g.actors), "gpus": self.owned[k], "calls": g.calls, "errors": g.errors, "seconds": round(g.seconds, 3)} for k, g in self.groups.items()}

    def close(self) -> None:
        for g in self.groups.values():
            g.close()
        self.groups.clear()


__all__ = ["WorkerPool", "WorkerGroup", "ThreadActor", "ProcessActor"]
