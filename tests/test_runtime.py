"""Distributed runtime: dispatch modes, handles over inline and multi-process (gloo) pools, failure detection on host ranks."""
import os
import sys
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _roles import Echo  # noqa: E402

from unirl_b200.distributed.group import DevicePool, Dispatch, Execute, WorkerDied, WorkerError, WorkerTimeout, placement, remote
from unirl_b200.distributed.group.dispatch import collect, plan_dispatch, resolve_backward_dispatch_mode
from unirl_b200.distributed.group.remote import make_rank_infos
from unirl_b200.distributed.tensor.grad_context import enable_grad
from unirl_b200.distributed.utils import Broadcast


def test_rank_layout_and_dispatch_plans():
    infos = make_rank_infos(8, tp=2, sp=2)
    assert infos[0].dp_size == 2 and [i.tp_rank for i in infos[:4]] == [0, 1, 0, 1] and [i.sp_rank for i in infos[:4]] == [0, 0, 1, 1]
    assert [i.dp_rank for i in infos] == [0, 0, 0, 0, 1, 1, 1, 1]
    x = torch.arange(4)
    shards = plan_dispatch(Dispatch.DP_SCATTER, infos, 2, (x,), {"k": Broadcast([1, 2, 3, 4])}, 4)
    assert all(torch.equal(s[0][0], x[:2]) for s in shards[:4]) and shards[5][1]["k"] == [1, 2, 3, 4]
    head = plan_dispatch(Dispatch.DP_SCATTER_HEAD, infos, 2, (x,), {}, 4)
    assert head[1] == ((), {}) and torch.equal(head[4][0][0], x[2:])
    sc = plan_dispatch(Dispatch.SCATTER, make_rank_infos(4), 4, (x,), {}, 4)
    assert [int(s[0][0]) for s in sc] == [0, 1, 2, 3]
    merged = collect(Dispatch.DP_SCATTER, infos, [torch.tensor([r]) for r in range(8)])
    assert merged.tolist() == [0, 4]
    with pytest.raises(ValueError):
        resolve_backward_dispatch_mode("f", Dispatch.BROADCAST, infos)
    with pytest.raises(ValueError):
        make_rank_infos(6, tp=4)


def test_inline_pool_scatter_localize_and_gc():
    pool = DevicePool(gpus_per_node=2, backend="inline", device="cpu")
    try:
        with placement(pool, num_devices=1):
            a = remote(Echo, scale=2.0)
        with placement(pool, num_devices=1):
            b = remote(Echo, scale=3.0)
        with pytest.raises(RuntimeError):
            with placement(pool, num_devices=1):
                pass
        out = a.run(torch.arange(4.0).view(4, 1))
        assert out["y"].refs[0].owner == 0 and out["n"] == [0, 0, 0, 0]
        out2 = b.run(out["y"])  # rows live on worker 0, consumer is worker 1 => one hop
        assert out2["y"].local().flatten().tolist() == [0.0, 6.0, 12.0, 18.0]
        assert b.only_zero() == ["zero"]
        with pytest.raises(RuntimeError, match="placement"):
            remote(Echo)
        del out, out2
        import gc

        gc.collect()
        assert all(s["tensors"] == 0 for s in pool.store_stats())
    finally:
        pool.shutdown()


def test_rpc_autograd_inline():
    pool = DevicePool(gpus_per_node=2, backend="inline", device="cpu")
    try:
        with placement(pool, devices=[0, 1]):
            h = remote(Echo)
        with enable_grad(h) as ctx:
            x = h.square(torch.tensor([[1.0], [2.0], [3.0], [4.0]]))
            y = h.square(x)
            y.grad = h.square(torch.ones(4, 1))  # seed dL/dy = 1 (any handle of the right shape)
            ctx.backward()
            assert x.grad is not None
            assert x.grad.local().flatten().tolist() == [2.0, 8.0, 18.0, 32.0]  # d(x^2)/dx at x = y_in
    finally:
        pool.shutdown()


@pytest.mark.timeout(300)
def test_mp_pool_collectives_errors_and_timeouts():
    pool = DevicePool(gpus_per_node=2, backend="mp", device="cpu", call_timeout_s=120)
    try:
        with placement(pool, devices=[0, 1]):
            c = remote(Echo, role_name="both")
        with placement(pool, devices=[1]):
            solo = remote(Echo, scale=3.0)
        assert c.who() == [0, 1] and c.allsum(1) == [3.0, 3.0]
        out = c.run(torch.arange(4.0).view(4, 1))
        assert [r.owner for r in out["y"].refs] == [0, 1]
        got = solo.run(out["y"])["y"].local().flatten().tolist()  # worker 0's rows hop to worker 1 over gloo
        assert got == [0.0, 3.0, 9.0, 12.0]
        # three fields of one producer consumed on another worker: they travel as one message per dtype, not one per tensor
        f = c.three(torch.arange(4.0).view(4, 1))
        before = pool.store_stats()[0]["messages_sent"]
        got = solo.combine(f["a"], f["b"], f["c"]).local().flatten().tolist()
        assert got == [0.0, 24.0, 48.0, 72.0]
        assert pool.store_stats()[0]["messages_sent"] - before == 2  # fp32 rows of a and b together, int64 rows of c
        with pytest.raises(WorkerError, match="boom from rank"):
            c.boom()
        with pytest.raises(WorkerTimeout, match="stall"):
            c._invoke("stall", Dispatch.BROADCAST, Execute.ALL, (3,), {}, timeout=0.5)
        time.sleep(3.0)
        assert c.who() == [0, 1], "pool must stay usable after a deadline expiry"
    finally:
        pool.shutdown()


@pytest.mark.timeout(300)
def test_mp_pool_detects_dead_worker():
    pool = DevicePool(gpus_per_node=2, backend="mp", device="cpu", call_timeout_s=60)
    try:
        with placement(pool, devices=[0, 1]):
            c = remote(Echo)
        pool.workers[1].proc.kill()  # host-side fault injection: the rank simply disappears between calls
        pool.workers[1].proc.join(10)
        with pytest.raises((WorkerDied, WorkerTimeout)):
            c.who()
    finally:
        pool.shutdown()


def test_tensor_meta_slice_cuts_through_a_handle_without_copy():
    """A DP=2 consumer of a DP=1 producer: the row range is a window of the single stored tensor."""
    from unirl_b200.distributed.tensor.transport import TensorMeta, WorkerLocalTransport

    tr = WorkerLocalTransport(0, torch.device("cpu"))
    full = torch.arange(64 * 3, dtype=torch.float32).reshape(64, 3)
    meta = TensorMeta.from_refs([tr.put(full[:40]), tr.put(full[40:])])
    a, b = meta.chunk(2)
    assert a.batch_size == b.batch_size == 32 and len(a.refs) == 1 and len(b.refs) == 2
    assert torch.equal(tr.get(a.refs), full[:32]) and torch.equal(tr.get(b.refs), full[32:])
    assert b.refs[0].base is not None and b.refs[0].lo == 32 and b.refs[1].base is None
    inner = b.slice(4, 12)  # window of a window
    assert torch.equal(tr.get(inner.refs), full[36:44])
    assert tr.get(a.refs).data_ptr() == tr.store.get(meta.refs[0].key).data_ptr()  # a view, not a copy
