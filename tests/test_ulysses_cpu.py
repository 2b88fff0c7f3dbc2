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


class _GlooHeadScatter:
    """Stand-in for the GEMM whose epilogue stores head tiles to their owners: same contract (``[B, l, K]`` → ``[parts, B, P·l, H/P, D]``
    in a buffer that is reused two calls later), the data moved by a library all-to-all.  Lets the model-side logic of the fused form
    (norm and rotary embedding after the exchange, text heads sliced, backward through the inverse exchange) run on CPU ranks."""

    def __init__(self, comm):
        self.comm, self.calls, self._bufs, self._flip = comm, 0, [None, None], 0

    def supports(self, x, weight, heads, head_dim):
        return True

    def project(self, x, weight, bias, heads, head_dim, parts=3, stat_parts=0):
        from unirl_b200.parallel.ulysses import _a2a_seq_to_head

        b, l, _ = x.shape
        y = x.reshape(b * l, -1) @ weight.t()
        if bias is not None:
            y = y + bias
        n_head_cols = parts * heads * head_dim
        rest = y[:, n_head_cols:].reshape(b, l, -1) if y.shape[1] > n_head_cols else None
        y = y[:, :n_head_cols].view(b, l, parts, heads, head_dim)
        sq = y[:, :, :stat_parts].float().pow(2).sum((-1, -2)).permute(2, 0, 1).contiguous() if stat_parts else None  # [stat_parts, B, l]
        out = torch.stack([_a2a_seq_to_head(y[:, :, i].contiguous(), self.comm) for i in range(parts)])
        i = self._flip
        self._flip ^= 1
        if self._bufs[i] is None or self._bufs[i].shape != out.shape:
            self._bufs[i] = torch.empty_like(out)
        self._bufs[i].copy_(out)  # reused like the symmetric receive buffers: a caller that keeps a view past the next call but one reads garbage
        self.calls += 1
        return (self._bufs[i], rest, sq) if stat_parts else (self._bufs[i], rest)


def _body_fused(rank, world):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.dit.modeling import DiTConfig, DiTTransformer
    from unirl_b200.parallel.ulysses import UlyssesContext

    out = {}
    for name, cfg in (("joint", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=3, num_single_blocks=0, text_dim=32, pooled_dim=24,
                                          rope_axes=(4, 6, 6), in_channels=4)),
                      ("joint+single", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=1, num_single_blocks=2, text_dim=32, pooled_dim=24,
                                                 rope_axes=(4, 6, 6), in_channels=4)),
                      ("joint-sincos", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=3, text_dim=32, pooled_dim=24, pos_embed="sincos2d",
                                                 pos_embed_max_size=8, dual_attention_blocks=(0,), in_channels=4)),
                      ("cross-video", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=0, num_cross_blocks=3, text_dim=32, pooled_dim=0,
                                                rope_axes=(4, 6, 6), in_channels=4, is_video=True)),
                      ("cross-video-norm-over-heads", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=0, num_cross_blocks=3, text_dim=32, pooled_dim=0,
                                                                rope_axes=(4, 6, 6), in_channels=4, is_video=True, qk_norm_scope="full"))):
        torch.manual_seed(0)
        ref = DiTTransformer(cfg, dtype=torch.float32).init_weights(1)
        if cfg.qk_norm_scope == "full":  # norm scales away from one, so that the weight slices and their gradients are really exercised
            with torch.no_grad():
                for n, p in ref.named_parameters():
                    if n.endswith(("q_norm", "k_norm")):
                        p.add_(torch.randn_like(p) * 0.2)
        ctx = UlyssesContext(Comm.world())
        ctx._scatter, ctx._scatter_tried, ctx.fuse_projection_norm_over_heads = _GlooHeadScatter(ctx.comm), True, True
        sp = DiTTransformer(cfg, dtype=torch.float32, sp=ctx).init_weights(1)
        sp.load_state_dict(ref.state_dict())
        x = torch.randn(2, 4, 3, 8, 8) if cfg.is_video else torch.randn(2, 4, 8, 8)
        t, txt = torch.tensor([700.0, 100.0]), torch.randn(2, 5, 32)
        pooled = torch.randn(2, 24) if cfg.pooled_dim else None
        a, b = ref(x, t, txt, pooled), sp(x, t, txt, pooled)
        a.square().mean().backward()
        b.square().mean().backward()
        ga = torch.cat([p.grad.flatten() for p in ref.parameters() if p.grad is not None])
        gb = torch.cat([p.grad.flatten() for p in sp.parameters() if p.grad is not None])
        out[name] = (float((a - b).abs().max()), ga, gb, ctx._scatter.calls)
    return out


def test_sequence_parallel_with_exchange_inside_the_projection_matches_single_rank():
    """The fused form of the attention input (projection that delivers head shards, q / k norm and rotary embedding after the exchange)
    against the single-rank model, forward and every gradient; the projection's data movement is played by a library all-to-all here."""
    r0, r1 = run_ranks(_body_fused, 2)
    for name in r0:
        assert r0[name][3] >= 3, (name, r0[name][3])  # the fused form was taken in every block
        assert r0[name][0] < 1e-5 and r1[name][0] < 1e-5, (name, r0[name][0])
        ga, g0, g1 = r0[name][1], r0[name][2], r1[name][2]
        summed = g0 + g1
        ok = ((summed - ga).abs() < 1e-4) | (((g0 - ga).abs() < 1e-4) & ((g1 - ga).abs() < 1e-4))
        assert bool(ok.all()), (name, int((~ok).sum()), ok.numel())


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
