"""Expert parallelism on 2 gloo ranks: the sharded MoE layer equals the replicated one in forward, backward and training."""
import torch

from _spawn import run_ranks


def _module_body(rank, world):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.unified.modeling import MoEFFN, UnifiedConfig
    from unirl_b200.parallel.expert_parallel import ExpertParallelContext

    cfg = UnifiedConfig.tiny()
    torch.manual_seed(0)
    ref = MoEFFN(cfg, torch.float32, "cpu")
    for p in ref.parameters():
        torch.nn.init.normal_(p, std=0.1)
    ep = MoEFFN(cfg, torch.float32, "cpu")
    ep.load_state_dict(ref.state_dict())
    ep.shard_experts(ExpertParallelContext(Comm.world()))
    assert len(ep.experts) == cfg.num_experts // world
    torch.manual_seed(10 + rank)
    x = torch.randn(6, cfg.hidden_size)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = ref(xa), ep(xb)
    ya.square().sum().backward()
    yb.square().sum().backward()
    lo = rank * (cfg.num_experts // world)
    g_all = torch.stack([e.gate_up.grad if e.gate_up.grad is not None else torch.zeros_like(e.gate_up) for e in ref.experts])
    torch.distributed.all_reduce(g_all)  # the replicated layer sees only this rank's tokens; the sharded one sees every rank's
    return (float((ya - yb).detach().abs().max()), float((xa.grad - xb.grad).abs().max()), float((g_all[lo] - ep.experts[0].gate_up.grad).abs().max()))


def test_expert_parallel_layer_matches_replicated_layer():
    for out, gx, gw in run_ranks(_module_body, 2):
        assert out < 1e-5 and gx < 1e-5 and gw < 1e-5


def _train_body(rank, world, use_ep):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.unified.modeling import UnifiedConfig, UnifiedTransformer
    from unirl_b200.parallel.expert_parallel import ExpertParallelContext
    from unirl_b200.parallel.flat_shard import FlatShardedModel

    torch.manual_seed(0)
    model = UnifiedTransformer(UnifiedConfig.tiny(), dtype=torch.float32).init_weights(0)
    comm = Comm.world()
    if use_ep:
        ctx = ExpertParallelContext(comm)
        for m in model.modules():
            if hasattr(m, "shard_experts"):
                m.shard_experts(ctx)
    sh = FlatShardedModel(model, comm, block_class_names=("UnifiedLayer",), low_dtype=torch.float32)
    assert any(g.expert_local for g in sh.groups) == use_ep
    g = torch.Generator().manual_seed(3)
    data = [torch.randint(3, 500, (world, 2, 9), generator=g) for _ in range(2)]
    for i in range(2):
        sh.zero_grad()
        sh.set_grad_sync(True)
        ids = data[i][rank]
        model.forward_text(ids, torch.ones_like(ids)).square().mean().backward()
        sh.finish_grad_sync()
        norm = sh.grad_norm()
        sh.optimizer_step(lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, step=i + 1, clip_coef=torch.clamp(1.0 / (norm + 1e-6), max=1.0).reshape(1))
    lo = rank * 2 if use_ep else 0
    experts = {f"{li}.{lo + j}": e.gate_up.detach().clone() for li, layer in enumerate(model.layers) for j, e in enumerate(layer.sets[0].ffn.experts)}
    return float(norm), model.layers[0].sets[0].qkv.detach().clone(), experts


def test_training_with_expert_parallel_groups_matches_replicated_experts():
    rep = run_ranks(_train_body, 2, False)
    ep = run_ranks(_train_body, 2, True)
    assert abs(rep[0][0] - ep[0][0]) < 1e-5
    torch.testing.assert_close(ep[0][1], rep[0][1], atol=2e-4, rtol=1e-3)  # Adam amplifies summation-order noise on near-zero gradients
    for r in range(2):
        for k, w in ep[r][2].items():
            torch.testing.assert_close(w, rep[0][2][k], atol=2e-4, rtol=1e-3)
