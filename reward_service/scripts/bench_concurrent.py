"""Throughput of a running reward service under concurrent clients:
``python bench_concurrent.py http://127.0.0.1:8077 clip --clients 8 --requests 32 --batch 8``."""
import argparse
import time
from concurrent.futures import ThreadPoolExecutor

import torch

from unirl_b200.reward.remote import RemoteRewardBackend
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.reward import RewardRequest

ap = argparse.ArgumentParser()
ap.add_argument("url")
ap.add_argument("scorer")
ap.add_argument("--clients", type=int, default=8)
ap.add_argument("--requests", type=int, default=32)
ap.add_argument("--batch", type=int, default=8)
a = ap.parse_args()
be = RemoteRewardBackend(a.url, scorers=[a.scorer], batch_size=a.batch, concurrency=1)
req = RewardRequest(primitives={"text": Texts.from_list(["a photo"] * a.batch)}, generated={"image": Images(pixels=torch.rand(a.batch, 3, 256, 256))},
                    sample_ids=[str(i) for i in range(a.batch)])
t0 = time.perf_counter()
with ThreadPoolExecutor(a.clients) as ex:
    list(ex.map(lambda _: be.compute_rewards(req), range(a.requests)))
dt = time.perf_counter() - t0
print(f"{a.requests * a.batch / dt:.1f} images/s over {a.clients} clients ({dt:.2f} s)")
