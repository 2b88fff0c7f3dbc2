"""Tensor-parallel DiT sampler on 2 gloo ranks: the sharded model's output equals the single-rank one for every block type, full tensors
arriving later (weight sync) are cut to the rank's shard, and LoRA adapters follow the shards."""
import torch

from _spawn import run_ranks


def _configs():
    from unirl_b200.models.dit.modeling import DiTConfig

    return (("joint+dual+single", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=2, num_single_blocks=2, text_dim=32, pooled_dim=24,
                                            rope_axes=(4, 6, 6), in_channels=4, dual_attention_blocks=(0,))),
            ("cross-video", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=0, num_cross_blocks=2, text_dim=32, pooled_dim=0,
                                      rope_axes=(4, 6, 6), in_channels=4, is_video=True)),
            ("cross-video-norm-over-heads", DiTConfig(hidden_size=64, num_heads=4, head_dim=16, num_joint_blocks=0, num_cross_blocks=2, text_dim=32, pooled_dim=0,
                                                      rope_axes=(4, 6, 6), in_channels=4, is_video=True, qk_norm_scope="full")))


def _inputs(cfg):
    torch.manual_seed(5)
    x = torch.randn(2, 4, 3, 8, 8) if cfg.is_video else torch.randn(2, 4, 8, 8)
    return x, torch.tensor([700.0, 100.0]), torch.randn(2, 5, 32), (torch.randn(2, 24) if cfg.pooled_dim else None)


def _body(rank, world):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.dit.modeling import DiTTransformer
    from unirl_b200.models.qwen3.modeling import TPContext
    from unirl_b200.train import inject

    comm = Comm.world()
    tp = TPContext(rank, world, lambda t: comm.all_reduce(t))
    out = {}
    for name, cfg in _configs():
        torch.manual_seed(0)
        ref = DiTTransformer(cfg, dtype=torch.float32).init_weights(1)
        with torch.no_grad():
            for n, p in ref.named_parameters():
                if p.dim() == 1:
                    p.add_(torch.randn_like(p) * 0.2)  # biases and norm scales away from their constant initial values
        full = {k: v.clone() for k, v in ref.state_dict().items()}
        model = DiTTransformer(cfg, dtype=torch.float32).init_weights(1)
        model.load_state_dict(full)
        model.apply_tensor_parallel(tp)
        x, t, txt, pooled = _inputs(cfg)
        with torch.no_grad():
            a, b = ref(x, t, txt, pooled), model(x, t, txt, pooled)
        row = {"fwd": float((a - b).abs().max()), "params": sum(p.numel() for p in model.parameters()) / sum(p.numel() for p in ref.parameters())}
        # weight sync: new FULL tensors arrive, every rank keeps its part
        new = {k: v + 0.01 * torch.randn(v.shape, generator=torch.Generator().manual_seed(11)) for k, v in full.items()}
        ref.load_state_dict(new)
        own = dict(model.named_parameters())
        with torch.no_grad():
            for k, v in new.items():
                if k in own:
                    own[k].copy_(model.tp_slice(k, v))
            row["fwd_after_sync"] = float((ref(x, t, txt, pooled) - model(x, t, txt, pooled)).abs().max())
        # adapters: trained on full shapes, installed on the shards
        inject.inject_lora(ref, rank=4, alpha=8.0, target_modules=("to_q", "to_v", "to_out.0", "ff.net.0.proj", "ff.net.2", "proj_mlp", "proj_out"), adapter_name="default", trainable=False,
                           freeze_base=True)
        inject.inject_lora(model, rank=4, alpha=8.0, target_modules=("to_q", "to_v", "to_out.0", "ff.net.0.proj", "ff.net.2", "proj_mlp", "proj_out"), adapter_name="default", trainable=False,
                           freeze_base=True)
        src = inject.lora_named_tensors(ref, "default", prefix="")
        g = torch.Generator().manual_seed(3)
        with torch.no_grad():
            for k, v in src.items():
                v.copy_(torch.randn(v.shape, generator=g) * 0.1)
            dst = inject.lora_named_tensors(model, "default", prefix="")
            assert set(dst) == set(src) and len(src) > 0
            for k, v in src.items():
                dst[k].copy_(model.tp_slice(k, v))
            row["fwd_lora"] = float((ref(x, t, txt, pooled) - model(x, t, txt, pooled)).abs().max())
            row["lora_tensors"] = len(src)
        out[name] = row
    return out


def test_tensor_parallel_dit_matches_single_rank():
    r0, r1 = run_ranks(_body, 2)
    for name in r0:
        for r in (r0, r1):
            # fp32 rounding only (measured 3e-8 .. 1e-7); a mis-sharded projection moves the output by 1e-5 or more in this set-up
            assert r[name]["fwd"] < 2e-6 and r[name]["fwd_after_sync"] < 2e-6 and r[name]["fwd_lora"] < 2e-6, (name, r[name])
            assert 0.5 < r[name]["params"] < 0.8 and r[name]["lora_tensors"] >= 4, (name, r[name])  # the blocks are halved, embedders and modulation stay whole


import pytest  # noqa: E402


@pytest.mark.timeout(600)
def test_trainer_with_tensor_parallel_sampler_engine_is_on_policy():
    """FlowGRPO on the tiny DiT, two gloo ranks: the trainer is data-parallel, the native sampler engine ONE replica split over both ranks
    (tp=2) with weights of its own, synchronised from the trainer's full tensors every step.  The first update is on-policy — the
    trainer's replay reproduces the sampler's log-probs — only if the sharded sampler computes what the unsharded model computes."""
    from test_diffusion_cpu import _trainer

    ov = ["num_devices=2", "pool_backend=mp", "+rollout_parallel={tp: 2}",
          "rollout._target_=unirl_b200.rollout.engine.native_diffusion.engine.NativeDiffusionRolloutEngine", "~rollout.stage_attrs",
          "+rollout.config={pipeline_cls: unirl_b200.models.sd3.pipeline.SD3Pipeline, pipeline_config_cls: unirl_b200.models.sd3.config.SD3PipelineConfig, "
          "pretrained_model_ckpt_path: 'random:tiny-sd3', model_precision: fp32, autocast_precision: fp32, device: cpu, share_trainer_weights: false, tp_size: 2}",
          "+sync={_target_: unirl_b200.distributed.weight_sync.full.tensor.TensorWeightSync}"]
    tr = _trainer(ov)
    try:
        tr.train(num_rollouts=2, weight_sync_interval=1)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2
        assert abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4 and abs(rows[1]["train/ratio_mean"] - 1.0) < 1e-4  # also after a weight sync into the shards
        sums = tr.rollout.compute_local_param_checksums()
        assert len(sums) == 2 and sums[0] != sums[1], "the two ranks hold different shards"
    finally:
        tr.shutdown()
