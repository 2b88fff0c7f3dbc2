"""Roles used by runtime tests (must be importable by spawned worker processes)."""
import torch

from unirl_b200.distributed.group import Dispatch, Execute, Remote, distributed


class Echo(Remote):
    def __init__(self, scale=1.0):
        super().__init__()
        self.scale = scale

    @distributed
    def run(self, x, tag=None):
        return {"y": x * self.scale + self.rank_info.rank, "n": [self.rank_info.rank] * x.shape[0]}

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def who(self):
        return self.rank_info.rank

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def allsum(self, v):
        t = torch.tensor([float(v + self.rank_info.rank)])
        self.comm.all_reduce(t)
        return float(t)

    @distributed(dispatch_mode=Dispatch.BROADCAST, execute_mode=Execute.RANK_ZERO)
    def only_zero(self):
        return "zero"

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def boom(self):
        raise ValueError("boom from rank %d" % self.rank_info.rank)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def stall(self, seconds):
        import time

        time.sleep(seconds)
        return True

    @distributed
    def square(self, x):
        return x * x

    @distributed
    def combine(self, a, b, c):
        """Three row-aligned inputs (two fp32, one int64): what a consumer of several fields of one producer looks like."""
        return a + 10.0 * b + c.to(a.dtype)

    @distributed
    def three(self, x):
        return {"a": x, "b": x * 2.0, "c": (x * 3.0).long()}
