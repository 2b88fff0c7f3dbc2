"""Context-parallel causal attention on gloo ranks equals single-rank attention, forward and backward, contiguous and zig-zag."""
import pytest
import torch

from _spawn import run_ranks


def _body(rank, world, zigzag):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.parallel.context_parallel import ContextParallel, reference_attention

    torch.manual_seed(0)
    B, L, Hq, Hkv, D = 2, 24, 4, 2, 8
    q, k, v = torch.randn(B, L, Hq, D), torch.randn(B, L, Hkv, D), torch.randn(B, L, Hkv, D)
    w = torch.randn(B, L, Hq, D)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    (reference_attention(qr, kr, vr) * w).sum().backward()
    cp = ContextParallel(Comm.world(), zigzag=zigzag)
    ql, kl, vl = (cp.shard_sequence(t).clone().requires_grad_() for t in (q, k, v))
    o = cp.attention(ql, kl, vl)
    (o * cp.shard_sequence(w)).sum().backward()
    full = cp.gather_sequence(o.detach())
    ref = reference_attention(q, k, v)
    idx = cp.token_index(L)
    return {"fwd": float((full - ref).abs().max()), "dq": float((ql.grad - qr.grad[:, idx]).abs().max()),
            "dk": float((kl.grad - kr.grad[:, idx]).abs().max()), "dv": float((vl.grad - vr.grad[:, idx]).abs().max())}


@pytest.mark.parametrize("world,zigzag", [(2, False), (2, True), (3, False)])
def test_context_parallel_attention_matches_single_rank(world, zigzag):
    for out in run_ranks(_body, world, zigzag):
        assert max(out.values()) < 1e-5, out
