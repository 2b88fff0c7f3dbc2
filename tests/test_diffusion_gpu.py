"""Diffusion stack on a B200: every DiT family generates in bf16 on CUDA (fused SDE kernels, dense attention, native GEMMs where
shapes qualify) and the training replay reproduces the rollout's log-probs; one Flow-DPPO trainer step with LoRA runs end to end."""
import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.models.dit import DiTConditions, DiTDiffusionParams, DiTPipeline, DiTPipelineConfig
from unirl_b200.trainer.diffusion import DiffusionTrainer
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.sampling import DiffusionSamplingParams

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,kw,video", [("tiny-sd3", {}, False), ("tiny-wan", {"num_frames": 9}, True), ("tiny-qwen-image", {}, False),
                                              ("tiny-flux2", {}, False), ("tiny-z-image", {}, False), ("tiny-hunyuan-video", {"num_frames": 5}, True)])
def test_family_generates_on_cuda_and_replay_tracks_rollout(preset, kw, video):
    pipe = DiTPipeline.from_config(DiTPipelineConfig(pretrained_model_ckpt_path=f"random:{preset}", model_precision="bf16", device="cuda"))
    sp = DiffusionSamplingParams(num_inference_steps=4, guidance_scale=3.0, height=64, width=64, seed=1, sde_indices=[1, 2], **kw)
    req = RolloutReq(sample_ids=["a/0", "a/1", "b/0"], group_ids=["a", "a", "b"], primitives={"text": Texts.from_list(["a cat", "a cat", "dog"])},
                     sampling_params=sp)
    tr = pipe.generate(req).tracks["diffusion"]
    seg = tr.segment
    assert seg.latents.is_cuda or seg.latents.device.type == "cpu"  # trajectories may be parked on the host
    assert seg.sde_logp.shape == (3, 2) and seg.latents.dim() == (6 if video else 5) and len(tr.decoded) == 3
    assert torch.isfinite(seg.latents.float()).all() and torch.isfinite(seg.sde_logp.float()).all()
    params = DiTDiffusionParams(guidance_scale=3.0, true_cfg=not pipe.bundle.model_config.guidance_embed)
    out = pipe.diffusion.replay(DiTConditions.from_dict(tr.conditions), segment=seg, params=params)
    assert out.log_probs.requires_grad
    # bf16 transformer on both sides; the SDE arithmetic is fp32: log-probs agree to bf16 noise of the velocity
    ref = seg.sde_logp.to(out.log_probs.device).float()
    assert float((out.log_probs.detach().float() - ref).abs().max()) <= 2e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.timeout(600)
def test_flowdppo_lora_trainer_step_on_cuda():
    cfg = compose("diffusion/tiny_sd3_flowgrpo_cpu", overrides=[
        "algorithm._target_=unirl_b200.algorithms.flowdppo.FlowDPPO", "~algorithm.clip_range", "~algorithm.old_logp_source", "pool_device=cuda",
        "bundle.config.model_precision=bf16", "bundle.config.device=cuda", "bundle.config.autocast_precision=bf16", "backend.fsdp_cfg.mixed_precision=true",
        "reward.backend.device=cuda"])
    tr = DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                          rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                          data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=None)
    try:
        before = tr.backend.compute_local_param_checksums()[0]
        tr.train(num_rollouts=2)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2 and all("train/policy_loss" in r for r in rows)
        assert tr.backend.compute_local_param_checksums()[0] != before, "no trainable parameter changed"
    finally:
        tr.shutdown()
