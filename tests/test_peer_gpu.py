"""Peer-memory collective kernels: single-device checks of the data path and of the bounded wait, and
two-rank runs (one CUDA device per rank, NCCL for plumbing, NVLS off) against library collectives."""
import pytest
import torch

from _spawn import run_ranks

pytestmark = pytest.mark.gpu

BIG = 1 << 30  # an epoch no kernel reaches: a pad pre-filled with it makes every wait pass at once


def _C():
    from unirl_b200.ops._ext import require_ext

    return require_ext()


def _local_comm(C, arenas, rank, preset, wait_s=5.0):
    """A world-of-len(arenas) communicator whose "peers" are buffers of this same device."""
    flags = [torch.full((64,), preset, dtype=torch.int32, device="cuda") for _ in arenas]
    state = torch.zeros(8, dtype=torch.int32, device="cuda")
    pc = C.PeerComm([a.data_ptr() for a in arenas], [f.data_ptr() for f in flags], rank, state, wait_s)
    return pc, flags, state


def test_allreduce_residual_rmsnorm_data_path_one_device():
    C = _C()
    torch.manual_seed(0)
    T, H, W = 37, 2560, 4
    arenas = [torch.randn(T * H, device="cuda").bfloat16() for _ in range(W)]
    res = torch.randn(T, H, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    want_x = (sum(a.float() for a in arenas).view(T, H) + res.float()).bfloat16()
    xf = want_x.float()
    want_h = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    outs = []
    for r in range(W):
        pc, flags, state = _local_comm(C, arenas, r, BIG)
        x, h = torch.empty(T, H, device="cuda", dtype=torch.bfloat16), torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        C.peer_allreduce_residual_rmsnorm(pc, arenas[r].view(T, H), res, w, x, h, 1e-6)
        torch.cuda.synchronize()
        assert int(state[4]) == 0 and int(state[0]) == 1  # no time-out; tick advanced once
        torch.testing.assert_close(x.float(), want_x.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(h.float(), want_h, atol=3e-2, rtol=2e-2)
        outs.append(x)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])  # every rank computes bit-identical sums


def test_reduce_scatter_and_adamw_publish_data_path_one_device():
    C = _C()
    from unirl_b200.ops.optim import adamw_reference

    torch.manual_seed(1)
    W, S = 2, 4096
    grads = [torch.randn(W * S, device="cuda") for _ in range(W)]
    want = sum(grads) / W
    shards = []
    for r in range(W):
        pc, _, state = _local_comm(C, grads, r, BIG)
        out, ss = torch.empty(S, device="cuda"), torch.zeros(1, device="cuda")
        C.peer_reduce_scatter_sumsq(pc, grads[r], out, ss, 1.0 / W)
        torch.cuda.synchronize()
        assert int(state[4]) == 0
        torch.testing.assert_close(out, want[r * S:(r + 1) * S], atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(ss[0], out.pow(2).sum(), rtol=1e-4, atol=1e-4)
        shards.append(out)
    replicas = [torch.zeros(W * S, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    clip = torch.tensor([0.5], device="cuda")
    for r in range(W):
        pc, _, state = _local_comm(C, replicas, r, BIG)
        master = torch.randn(S, device="cuda")
        m, v = torch.rand(S, device="cuda") * 0.1, torch.rand(S, device="cuda") * 0.01
        ref_p, ref_m, ref_v = master.clone(), m.clone(), v.clone()
        adamw_reference(ref_p, shards[r] * 0.5, ref_m, ref_v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
        C.peer_adamw_publish(pc, replicas[r], master, shards[r], m, v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, clip, 0.0)
        torch.cuda.synchronize()
        assert int(state[4]) == 0
        torch.testing.assert_close(master, ref_p, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(m, ref_m, atol=1e-6, rtol=1e-5)
        torch.testing.assert_close(v, ref_v, atol=1e-7, rtol=1e-5)
        for rep in replicas:  # the shard landed in EVERY replica
            torch.testing.assert_close(rep[r * S:(r + 1) * S].float(), ref_p.bfloat16().float(), atol=0, rtol=0)


def test_wait_runs_out_and_reports_status():
    """A flag that nothing sets: the kernel gives up after its budget, records the code and the context stays usable."""
    C = _C()
    arenas = [torch.zeros(1024, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    pc, flags, state = _local_comm(C, arenas, 0, 0, wait_s=0.3)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    C.peer_barrier(pc)
    t1.record()
    torch.cuda.synchronize()
    assert 250 < t0.elapsed_time(t1) < 5000
    assert int(state[4]) == 341  # entry wait of the barrier kernel on peer 1
    assert int(flags[1][0]) == 1  # the publish to the "peer" still happened
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


@pytest.mark.parametrize("mode", [0, 1])
def test_ulysses_exchange_data_path_one_device(mode):
    """Four "ranks" whose staged tensors live on this device: every rank's pull must equal the permutation of the library path."""
    C = _C()
    torch.manual_seed(4)
    W, B, l, Hp, D = 4, 2, 24, 3, 64
    shape = (B, l, W * Hp, D) if mode == 0 else (B, W * l, Hp, D)
    xs = [torch.randn(*shape, device="cuda").bfloat16() for _ in range(W)]
    arenas = [x.reshape(-1).clone() for x in xs]
    for r in range(W):
        pc, flags, state = _local_comm(C, arenas, r, BIG)
        out = C.peer_ulysses_exchange(pc, arenas[r], B, l, Hp, D, mode)
        torch.cuda.synchronize()
        assert int(state[4]) == 0 and int(state[0]) == 1
        if mode == 0:  # out[b, p*l + t, hh] = x_p[b, t, r*Hp + hh]
            want = torch.cat([x[:, :, r * Hp:(r + 1) * Hp] for x in xs], 1)
        else:          # out[b, t, p*Hp + hh] = x_p[b, r*l + t, hh]
            want = torch.cat([x[:, r * l:(r + 1) * l] for x in xs], 2)
        assert torch.equal(out, want), (mode, r)


@pytest.mark.parametrize("D,local_cols,bias", [(64, 0, True), (128, 256, True), (64, 128, False)])
def test_head_scatter_projection_data_path_one_device(D, local_cols, bias):
    """The QKV GEMM whose epilogue stores every head's columns into the rank that owns the head: four "ranks" whose receive buffers live on
    this device, run one after the other (the kernel itself never waits for a peer).  Each buffer must end up holding, for its heads,
    every rank's tokens at their place in the gathered sequence; trailing local columns come back as an ordinary matrix."""
    from unirl_b200.parallel.fused_collectives import FusedHeadScatterProjection as F

    C = _C()
    torch.manual_seed(5)
    W, B, l, heads, K = 4, 2, 200, 8, 512  # 400 rows per rank: three full 128-row tiles and a ragged one, rows crossing the batch boundary inside a tile
    hp, parts = heads // W, 3
    n = parts * heads * D + local_cols
    recv = [torch.full((parts * B * W * l * hp * D,), float("nan"), device="cuda").bfloat16() for _ in range(W)]
    xs = [(torch.randn(B, l, K, device="cuda") * 0.5).bfloat16() for _ in range(W)]
    w = (torch.randn(n, K, device="cuda") * 0.05).bfloat16()
    b = (torch.randn(n, device="cuda") * 0.1).bfloat16() if bias else None
    for r in range(W):
        table = F.pack_table(F.route_rows([t.data_ptr() for t in recv], r, W, B, l, heads, D, parts, n), "cuda")
        rest = C.gemm_bf16_route(xs[r].view(B * l, K), w, b, table, l, local_cols)
        torch.cuda.synchronize()
        assert C.gemm_status(True) == 0
        y = xs[r].view(B * l, K).float() @ w.float().t() + (b.float() if bias else 0.0)
        if local_cols:
            torch.testing.assert_close(rest.float(), y[:, n - local_cols:], atol=3e-2, rtol=2e-2)
        else:
            assert rest.numel() == 0
    for dst in range(W):
        got = recv[dst].view(parts, B, W * l, hp, D).float()
        assert not torch.isnan(got).any(), "every element of the receive buffer is written exactly by its owner"
        for src in range(W):
            y = (xs[src].view(B * l, K).float() @ w.float().t() + (b.float() if bias else 0.0))[:, : parts * heads * D].view(B, l, parts, heads, D)
            want = y[:, :, :, dst * hp:(dst + 1) * hp].permute(2, 0, 1, 3, 4)  # [parts, B, l, hp, D]
            torch.testing.assert_close(got[:, :, src * l:(src + 1) * l], want, atol=3e-2, rtol=2e-2)


def test_scatter_copy_table():
    from unirl_b200.distributed.weight_sync.full.reshard import CopyOp, execute_copy
    from unirl_b200.parallel.fused_collectives import reshard_scatter_local

    torch.manual_seed(2)
    src = torch.randn(64 * 96, device="cuda").bfloat16()
    dst_a, dst_b = torch.zeros(64 * 48, device="cuda", dtype=torch.bfloat16), torch.zeros(37, device="cuda", dtype=torch.bfloat16)
    plan = [(src, dst_a, CopyOp("w", 0, 48, 0, 64, 48, 96, 48)), (src, dst_b, CopyOp("b", 0, 5, 0, 1, 37, 37, 37))]
    assert reshard_scatter_local(plan)
    ra, rb = torch.zeros_like(dst_a), torch.zeros_like(dst_b)
    execute_copy(plan[0][2], src, ra)
    execute_copy(plan[1][2], src, rb)
    assert torch.equal(dst_a, ra) and torch.equal(dst_b, rb)


# ------------------------------------------------------------------------------------------------ two ranks
def _two_rank_body(rank, world):
    import torch.distributed as dist

    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.parallel.fused_collectives import FusedAllReduce, FusedShardComm
    from unirl_b200.parallel.flat_shard import FlatShardedModel, ShardComm

    dev = torch.device("cuda", rank)
    comm = Comm.world()
    out = {}
    # -- TP projection + all-reduce + residual + norm, many calls (both staging halves, epochs advance)
    torch.manual_seed(0)
    T, K, H = 48, 512, 1024
    w_full = torch.randn(H, K * world, device=dev).bfloat16() * 0.05
    x_full = torch.randn(T, K * world, device=dev).bfloat16()
    res = torch.randn(T, H, device=dev).bfloat16()
    nw = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    far = FusedAllReduce(comm, 64, H, dev, wait_s=10.0)
    errs = []
    for it in range(5):
        xs = (x_full * (it + 1)).bfloat16()
        x, h = far.proj_reduce_norm(xs[:, rank * K:(rank + 1) * K].contiguous(), w_full[:, rank * K:(rank + 1) * K].contiguous(), res, nw, 1e-6)
        y = torch.matmul(xs[:, rank * K:(rank + 1) * K], w_full[:, rank * K:(rank + 1) * K].t()).float()
        dist.all_reduce(y)
        want = y + res.float()
        errs.append(float((x.float() - want).abs().max() / want.abs().max()))
        hw = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        errs.append(float((h.float() - hw).abs().max() / hw.abs().max()))
    far.align()
    far.arena.check()
    out["ar_err"] = max(errs)
    # -- sharded trainer: fused vs library collectives on the same toy model
    def build(fused):
        torch.manual_seed(3)
        m = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 256)).to(dev).bfloat16()
        return m, FlatShardedModel(m, comm, block_class_names=("Linear",), shard_comm=FusedShardComm(comm, wait_s=10.0) if fused else ShardComm(comm))
    results = []
    for fused in (False, True):
        m, sh = build(fused)
        for step in range(3):
            sh.zero_grad()
            sh.set_grad_sync(True)
            torch.manual_seed(100 + step * world + rank)
            xb = torch.randn(32, 256, device=dev).bfloat16()
            m(xb).float().pow(2).mean().backward()
            sh.finish_grad_sync()
            norm = sh.grad_norm()
            coef = torch.clamp(1.0 / (norm + 1e-6), max=1.0).float().reshape(1)
            sh.optimizer_step(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, step=step + 1, clip_coef=coef)
            sh.shard_comm.check()
        torch.cuda.synchronize()
        results.append((float(norm), torch.cat([p.detach().float().reshape(-1) for p in m.parameters()]).cpu()))
    out["norm_nccl"], out["norm_fused"] = results[0][0], results[1][0]
    out["param_diff"] = float((results[0][1] - results[1][1]).abs().max())
    gathered = [torch.zeros_like(results[1][1]) for _ in range(world)]
    dist.all_gather_object(gathered, results[1][1])
    out["replica_diff"] = float(max((g - gathered[0]).abs().max() for g in gathered))
    # -- Ulysses attention: peer-memory exchange kernel vs pack + all-to-all + unpack, forward and backward
    from unirl_b200.parallel.ulysses import UlyssesContext

    torch.manual_seed(7 + rank)
    B, l, Hh, D, n_text = 2, 96, 8, 64, 5
    base = [torch.randn(B, n_text + l, Hh, D, device=dev).bfloat16() for _ in range(3)]
    if n_text:  # text rows are replicated on every rank
        for t in base:
            t0 = t[:, :n_text].clone()
            dist.broadcast(t0, 0)
            t[:, :n_text] = t0
    got = {}
    for kind in ("nccl", "fused"):
        ctx = UlyssesContext(comm, collectives=kind)
        q, k, v = (t.clone().requires_grad_() for t in base)
        o = ctx.attention(q, k, v, n_text)
        (o.float() * torch.linspace(0.5, 1.5, o.numel(), device=dev).view_as(o)).sum().backward()
        got[kind] = (o.detach().float(), q.grad.float(), k.grad.float(), v.grad.float())
        if kind == "fused":
            assert ctx._fused is not None, "the peer-memory exchange was not used"
            ctx._fused.check()
    out["ulysses_diff"] = float(max((a - b).abs().max() for a, b in zip(got["nccl"], got["fused"])))
    # -- the same exchange done by the QKV projection's own epilogue: a joint-block DiT under sequence parallelism, fused vs library form
    from unirl_b200.models.dit.modeling import DiTConfig, DiTTransformer

    cfg = DiTConfig(hidden_size=512, num_heads=8, head_dim=64, num_joint_blocks=2, num_single_blocks=0, text_dim=64, pooled_dim=32, rope_axes=(16, 24, 24), in_channels=4)
    res = {}
    for kind in ("nccl", "fused"):
        ctx = UlyssesContext(comm, collectives=kind)
        torch.manual_seed(21)
        model = DiTTransformer(cfg, dtype=torch.bfloat16, device=dev, sp=ctx).init_weights(1)
        torch.manual_seed(22)
        lat, tt, txt, pooled = torch.randn(2, 4, 64, 64, device=dev), torch.tensor([700.0, 100.0], device=dev), torch.randn(2, 7, 64, device=dev), torch.randn(2, 32, device=dev)
        y = model(lat, tt, txt, pooled)
        y.float().square().mean().backward()
        g = torch.cat([p.grad.float().flatten() for p in model.parameters() if p.grad is not None])
        res[kind] = (y.detach().float(), g)
        if kind == "fused":
            assert ctx._scatter is not None and ctx._scatter.calls >= 2, "the projection with the exchange in its epilogue was not used"
            ctx._scatter.check()
            with torch.no_grad():  # inference form: the attention reads the symmetric receive buffers in place
                y2 = model(lat, tt, txt, pooled)
            out["scatter_infer_diff"] = float((y2.float() - res[kind][0]).abs().max())
    scale = float(res["nccl"][0].abs().max())
    out["scatter_fwd_rel"] = float((res["nccl"][0] - res["fused"][0]).abs().max()) / scale
    out["scatter_grad_rel"] = float((res["nccl"][1] - res["fused"][1]).abs().max()) / float(res["nccl"][1].abs().max())
    return out


@pytest.mark.multigpu
def test_two_rank_fused_collectives_match_library():
    outs = run_ranks(_two_rank_body, 2, cuda=True, timeout=300)
    for o in outs:
        assert o["ar_err"] < 2e-2, o
        assert abs(o["norm_nccl"] - o["norm_fused"]) <= 1e-3 * max(1.0, o["norm_nccl"]), o
        assert o["param_diff"] <= 1e-2, o  # bf16 replicas after 3 steps
        assert o["replica_diff"] == 0.0, o  # every rank holds the same replica
        assert o["ulysses_diff"] == 0.0, o  # the exchange only moves data: both paths must agree bit for bit
        # q / k norm and rotary embedding run after the exchange in the fused form and the bias is added in fp32 before rounding: bf16-level agreement
        assert o["scatter_fwd_rel"] < 3e-2 and o["scatter_grad_rel"] < 5e-2 and o["scatter_infer_diff"] == 0.0, o


def test_gemm_with_allreduce_epilogue_data_path_one_device():
    """The GEMM whose epilogue pushes its partial into every rank's staging area and sums all partials: data path on one device (the
    "ranks" are arenas of this device, run one after the other; their flag areas are pre-filled so that no rank waits)."""
    C = _C()
    torch.manual_seed(3)
    W, M, N, K = 4, 96, 2560, 1024
    slot = 128 * N
    stage_elems, flag_words = 2 * W * slot, W * 1024
    arenas = [torch.zeros(stage_elems * 2 + flag_words * 4 + 256, dtype=torch.uint8, device="cuda") for _ in range(W)]
    stages = [a[: stage_elems * 2].view(torch.bfloat16) for a in arenas]
    flags = [a[stage_elems * 2 : stage_elems * 2 + flag_words * 4].view(torch.int32) for a in arenas]
    for f in flags:
        f.fill_(BIG)
    xs = [(torch.randn(M, K, device="cuda") * 0.3).bfloat16() for _ in range(W)]
    ws = [(torch.randn(N, K, device="cuda") * 0.05).bfloat16() for _ in range(W)]
    res = torch.randn(M, N, device="cuda").bfloat16()
    want = sum((x.float() @ w.float().t()).bfloat16().float() for x, w in zip(xs, ws)) + res.float()
    outs = []
    for rnd in range(2):  # first round fills every slot; second round (fresh epoch words) sees all partials
        for r in range(W):
            state = torch.zeros(8, dtype=torch.int32, device="cuda")
            pad = torch.full((64,), BIG, dtype=torch.int32, device="cuda")
            pc = C.PeerComm([a.data_ptr() for a in arenas], [pad.data_ptr()] * W, r, state, 5.0)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            C.gemm_skinny_allreduce(pc, stages[r], flags[r], xs[r], ws[r], res, out)
            torch.cuda.synchronize()
            assert int(state[4]) == 0 and int(state[0]) == 1, "no wait may time out; the epoch word advances by one"
            if rnd == 1:
                outs.append(out)
    for out in outs:
        _close = (out.float() - want).abs().max().item()
        assert _close < 0.1, _close
        assert torch.equal(out, outs[0]), "every rank must produce the same bits"


def _gemm_allreduce_body(rank, world):
    import torch.distributed as dist

    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.parallel.fused_collectives import FusedAllReduce

    dev = torch.device("cuda", rank)
    comm = Comm.world()
    H, K = 2560, 2048
    import os

    os.environ["UNIRL_B200_TP_FUSED_GEMM_MAX_M"] = "256"  # exercise the two-tile case as well
    far = FusedAllReduce(comm, max_tokens=512, hidden=H, device=dev, wait_s=10.0)
    out = {"max_err": 0.0, "rank_diff": 0.0, "fused_calls": 0}
    torch.manual_seed(11 + rank)
    w = (torch.randn(H, K, device=dev) * 0.05).bfloat16()
    nw = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    dist.broadcast(nw, 0)
    for T in (1, 64, 128, 200, 256):
        for rep in range(3):  # consecutive calls alternate the staging halves
            x = (torch.randn(T, K, device=dev) * 0.3).bfloat16()
            res = torch.randn(T, H, device=dev).bfloat16()
            dist.broadcast(res, 0)
            xo, ho = far.proj_reduce_norm(x, w, res, nw, 1e-6)
            ref = (x.float() @ w.float().t()).bfloat16().float()
            dist.all_reduce(ref)
            ref = ref + res.float()
            out["max_err"] = max(out["max_err"], float((xo.float() - ref).abs().max()))
            gathered = [torch.empty_like(xo) for _ in range(world)]
            dist.all_gather(gathered, xo)
            out["rank_diff"] = max(out["rank_diff"], max(float((g.float() - xo.float()).abs().max()) for g in gathered))
            hf = xo.float()
            href = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
            out["max_err"] = max(out["max_err"], float((ho.float() - href).abs().max()) * 0.5)
    far.arena.check()
    out["fused_calls"] = far.fused_calls
    return out


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_with_allreduce_epilogue_matches_library(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    outs = run_ranks(_gemm_allreduce_body, world, cuda=True, timeout=300)
    for o in outs:
        assert o["fused_calls"] == 15, o  # every call went through the GEMM with the all-reduce epilogue
        assert o["max_err"] < 0.15, o
        assert o["rank_diff"] == 0.0, o  # tensor-parallel ranks must hold identical activations


def _head_scatter_body(rank, world):
    """Projection with the exchange in its epilogue on real peers: every element against projection + library all-to-all, several calls in
    a row (both receive buffers, the rendezvous between them), two geometries; then a sequence-parallel DiT forward / backward both ways."""
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.dit.modeling import DiTConfig, DiTTransformer
    from unirl_b200.parallel.fused_collectives import FusedHeadScatterProjection
    from unirl_b200.parallel.ulysses import UlyssesContext, _a2a_seq_to_head

    dev = torch.device("cuda", rank)
    comm = Comm.world()
    sc = FusedHeadScatterProjection(comm, dev, wait_s=10.0)
    out = {"max_err": 0.0, "calls": 0}
    torch.manual_seed(31)
    for heads, D, B, l, K, extra in ((8, 64, 2, 136, 256, 0), (16, 128, 1, 200, 512, 128)):
        w = (torch.randn(3 * heads * D + extra, K, device=dev) * 0.05).bfloat16()  # same on every rank (same seed)
        b = (torch.randn(3 * heads * D + extra, device=dev) * 0.1).bfloat16()
        for rep in range(3):
            torch.manual_seed(100 * rep + rank)
            x = (torch.randn(B, l, K, device=dev) * 0.5).bfloat16()
            got, rest = sc.project(x, w, b, heads, D, 3)
            y = (x.view(B * l, K).float() @ w.float().t() + b.float()).bfloat16()
            parts = y[:, : 3 * heads * D].view(B, l, 3, heads, D)
            want = torch.stack([_a2a_seq_to_head(parts[:, :, i].contiguous(), comm) for i in range(3)])
            out["max_err"] = max(out["max_err"], float((got.float() - want.float()).abs().max()))
            if extra:
                out["max_err"] = max(out["max_err"], float((rest.view(B * l, extra).float() - y[:, 3 * heads * D:].float()).abs().max()))
    sc.align()
    sc.check()
    out["calls"] = sc.calls
    cfg = DiTConfig(hidden_size=512, num_heads=8, head_dim=64, num_joint_blocks=3, num_single_blocks=0, text_dim=64, pooled_dim=32, rope_axes=(16, 24, 24), in_channels=4)
    res = {}
    for kind in ("nccl", "fused"):
        ctx = UlyssesContext(comm, collectives=kind)
        torch.manual_seed(21)
        model = DiTTransformer(cfg, dtype=torch.bfloat16, device=dev, sp=ctx).init_weights(1)
        torch.manual_seed(22)
        lat, tt, txt, pooled = torch.randn(2, 4, 64, 64, device=dev), torch.tensor([700.0, 100.0], device=dev), torch.randn(2, 7, 64, device=dev), torch.randn(2, 32, device=dev)
        y = model(lat, tt, txt, pooled)
        y.float().square().mean().backward()
        res[kind] = (y.detach().float(), torch.cat([p.grad.float().flatten() for p in model.parameters() if p.grad is not None]))
        if kind == "fused":
            out["dit_calls"] = ctx._scatter.calls if ctx._scatter is not None else 0
            ctx._scatter.check()
    out["dit_fwd_rel"] = float((res["nccl"][0] - res["fused"][0]).abs().max()) / float(res["nccl"][0].abs().max())
    out["dit_grad_rel"] = float((res["nccl"][1] - res["fused"][1]).abs().max()) / float(res["nccl"][1].abs().max())
    return out


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_projection_with_exchange_in_epilogue_matches_library(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    outs = run_ranks(_head_scatter_body, world, cuda=True, timeout=300)
    for o in outs:
        assert o["calls"] == 6 and o["dit_calls"] >= 3, o
        assert o["max_err"] <= 2 ** -6, o  # one bf16 rounding step at the magnitudes involved: the bias is added in fp32 before rounding here, after it in the comparison
        assert o["dit_fwd_rel"] < 3e-2 and o["dit_grad_rel"] < 5e-2, o
