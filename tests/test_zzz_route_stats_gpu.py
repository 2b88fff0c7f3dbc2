"""Row statistics of the routed projection (the sum of squares an RMS norm over all heads of a token needs), one device.

Kept in a file of its own, sorted after the others: the statistic is the newest part of the GEMM's routed epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_routed_projection_row_statistics_one_device():
    from unirl_b200.ops._ext import require_ext
    from unirl_b200.parallel.fused_collectives import FusedHeadScatterProjection as F

    C = require_ext()
    torch.manual_seed(9)
    W, B, l, heads, D, K, local_cols = 2, 2, 200, 8, 64, 256, 128
    hp, parts = heads // W, 3
    n = parts * heads * D + local_cols
    recv = [torch.zeros(parts * B * W * l * hp * D, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    x = (torch.randn(B, l, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, K, device="cuda") * 0.05).bfloat16()
    b = (torch.randn(n, device="cuda") * 0.1).bfloat16()
    table = F.pack_table(F.route_rows([t.data_ptr() for t in recv], 0, W, B, l, heads, D, parts, n, stat_parts=2), "cuda")
    rowsq = torch.zeros(2, B * l, device="cuda")
    rest = C.gemm_bf16_route(x.view(B * l, K), w, b, table, l, local_cols, rowsq)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    y = (x.view(B * l, K).float() @ w.float().t() + b.float()).bfloat16().float()
    want = torch.stack([y[:, : heads * D].pow(2).sum(1), y[:, heads * D : 2 * heads * D].pow(2).sum(1)])
    torch.testing.assert_close(rowsq, want, rtol=5e-3, atol=1e-3)
    torch.testing.assert_close(rest.float(), y[:, n - local_cols:], atol=3e-2, rtol=2e-2)
    # the statistic is optional: without it the same call leaves the data path unchanged
    got = [t.clone() for t in recv]
    for t in recv:
        t.zero_()
    C.gemm_bf16_route(x.view(B * l, K), w, b, F.pack_table(F.route_rows([t.data_ptr() for t in recv], 0, W, B, l, heads, D, parts, n), "cuda"), l, local_cols)
    torch.cuda.synchronize()
    for a, c in zip(got, recv):
        assert torch.equal(a, c)
