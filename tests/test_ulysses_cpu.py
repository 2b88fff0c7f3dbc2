"""Ulysses sequence parallelism on 2 gloo ranks: the sharded DiT forward / backward equals the single-rank one."""
import torch

from _spawn import run_ranks


def _body(rank, world):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.dit.modeling import DiTConfig, DiTTransformer
    from unirl_b200.parallel.ulysses import UlyssesContext

    out = {}
    for name, cfg in (("joint+single", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=1, num_single_blocks=1, text_dim=32, pooled_dim=24,
                                                 rope_axes=(4, 6, 6), in_channels=4)),
                      ("cross-video", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=0, num_cross_blocks=2, text_dim=32, pooled_dim=0,
                                                rope_axes=(4, 6, 6), in_channels=4, is_video=True))):
        torch.manual_seed(0)
        ref = DiTTransformer(cfg, dtype=torch.float32).init_weights(1)
        sp = DiTTransformer(cfg, dtype=torch.float32, sp=UlyssesContext(Comm.world())).init_weights(1)
        x = torch.randn(2, 4, 3, 8, 8) if cfg.is_video else torch.randn(2, 4, 8, 8)
        t, txt = torch.tensor([700.0, 100.0]), torch.randn(2, 5, 32)
        pooled = torch.randn(2, 24) if cfg.pooled_dim else None
        a, b = ref(x, t, txt, pooled), sp(x, t, txt, pooled)
        a.square().mean().backward()
        b.square().mean().backward()
        ga = torch.cat([p.grad.flatten() for p in ref.parameters() if p.grad is not None])
        # latent-stream parameters see only this rank's tokens: their gradients add up over ranks; text-stream ones are replicated
        gb = torch.cat([p.grad.flatten() for p in sp.parameters() if p.grad is not None])
        out[name] = (float((a - b).abs().max()), ga, gb)
    return out


def test_sequence_parallel_dit_matches_single_rank():
    r0, r1 = run_ranks(_body, 2)
    for name in r0:
        assert r0[name][0] < 1e-5 and r1[name][0] < 1e-5, (name, r0[name][0])
        ga, g0, g1 = r0[name][1], r0[name][2], r1[name][2]
        summed = g0 + g1
        # every gradient entry equals the reference either as the rank sum (sharded-token path) or as each rank's own value (replicated path)
        ok = ((summed - ga).abs() < 1e-4) | (((g0 - ga).abs() < 1e-4) & ((g1 - ga).abs() < 1e-4))
        assert bool(ok.all()), (name, int((~ok).sum()), ok.numel())


def test_diffusion_trainer_with_sequence_parallel_ranks_matches_single_rank():
    """FlowGRPO on the tiny DiT: one process vs. two gloo ranks forming ONE sequence-parallel replica (sp=2, dp=1)."""
    from test_diffusion_cpu import _trainer

    def run(ov):
        tr = _trainer(ov)
        try:
            req = tr._build_req(tr.data_source.get_samples(tr.batch_size), 0)
            result, _reward = tr.train_step(req, rollout_id=0)
            row = [r for r in tr.wandb_logger.history if "train/step" in r][0]
            return {**row, "train/grad_norm": float(result.grad_norm)}
        finally:
            tr.shutdown()

    one = run([])
    two = run(["num_devices=2", "pool_backend=mp", "+train_parallel={sp: 2}", "+backend.fsdp_cfg.sp_size=2", "+rollout_parallel={sp: 2}"])
    assert abs(two["train/ratio_mean"] - 1.0) < 1e-4
    assert abs(one["train/policy_loss"] - two["train/policy_loss"]) < 1e-5 + 1e-3 * abs(one["train/policy_loss"])
    assert abs(one["train/grad_norm"] - two["train/grad_norm"]) < 1e-3 * max(1e-6, abs(one["train/grad_norm"])) + 1e-6
