"""Send one random image to a running reward service and print the scores: ``python smoke_client.py http://127.0.0.1:8077 clip,aesthetic``."""
import sys

import torch

from unirl_b200.reward.remote import RemoteRewardBackend
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.reward import RewardRequest

url, names = sys.argv[1], sys.argv[2].split(",") if len(sys.argv) > 2 else ["clip"]
be = RemoteRewardBackend(url, scorers=names)
out = be.compute_rewards(RewardRequest(primitives={"text": Texts.from_list(["a photo of a cat"])}, generated={"image": Images(pixels=torch.rand(1, 3, 64, 64))}, sample_ids=["0"]))
print(out.rewards, out.component_rewards)
