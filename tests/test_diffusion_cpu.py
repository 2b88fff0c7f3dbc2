"""Diffusion stack on CPU: every DiT family end to end (prompt → trajectory → decoded media), bit-exact rollout/replay
alignment, and the training loop with FlowGRPO, Flow-DPPO and DiffusionNFT (LoRA + EMA shadow adapter)."""
import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.models.dit import DiTConditions, DiTDiffusionParams, DiTPipeline, DiTPipelineConfig
from unirl_b200.trainer.diffusion import DiffusionTrainer
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.sampling import DiffusionSamplingParams


def _pipe(preset, cls=DiTPipeline, cfg_cls=DiTPipelineConfig, **kw):
    return cls.from_config(cfg_cls(pretrained_model_ckpt_path=f"random:{preset}", model_precision="fp32", device="cpu", autocast_precision="fp32", **kw))


def _req(**kw):
    sp = DiffusionSamplingParams(num_inference_steps=4, guidance_scale=3.0, height=64, width=64, seed=1, sde_indices=[1, 2], **kw)
    return RolloutReq(sample_ids=["a/0", "a/1", "b/0"], group_ids=["a", "a", "b"], primitives={"text": Texts.from_list(["a cat", "a cat", "dog"])},
                      sampling_params=sp)


@pytest.mark.parametrize("preset,kw,video", [("tiny-sd3", {}, False), ("tiny-wan", {"num_frames": 9}, True), ("tiny-qwen-image", {}, False),
                                              ("tiny-flux2", {}, False), ("tiny-z-image", {}, False), ("tiny-hunyuan-video", {"num_frames": 5}, True)])
def test_family_generates_and_replay_reproduces_rollout(preset, kw, video):
    pipe = _pipe(preset)
    tr = pipe.generate(_req(**kw)).tracks["diffusion"]
    seg = tr.segment
    assert seg.indices.tolist() == [1, 2, 3, 4] and seg.sde_indices.tolist() == [1, 2] and seg.sde_logp.shape == (3, 2)
    assert seg.latents.dim() == (6 if video else 5) and len(tr.decoded) == 3
    assert torch.isfinite(seg.latents).all() and torch.isfinite(seg.sde_logp).all()
    params = DiTDiffusionParams(guidance_scale=3.0, true_cfg=not pipe.bundle.model_config.guidance_embed)
    out = pipe.diffusion.replay(DiTConditions.from_dict(tr.conditions), segment=seg, params=params)
    assert float((out.log_probs.detach() - seg.sde_logp).abs().max()) < 1e-5 and float((out.prev_sample_means.detach() - seg.sde_means).abs().max()) < 1e-5
    assert out.log_probs.requires_grad


def test_same_group_shares_initial_noise_and_rebatching_is_deterministic():
    pipe = _pipe("tiny-sd3")
    full = pipe.generate(_req(init_same_noise=True)).tracks["diffusion"].segment
    req = _req(init_same_noise=True)
    part = pipe.generate(req.slice(1, 3)).tracks["diffusion"].segment  # samples a/1 and b/0 alone
    assert torch.allclose(full.latents[1:], part.latents, atol=1e-5), "per-sample seeds make trajectories independent of batching"
    x1 = pipe.generate(_req(init_same_noise=True, eta=0.0)).tracks["diffusion"].segment
    assert x1.sde_logp is None  # eta = 0: pure ODE, nothing to score


def test_sd3_diffusers_key_bridge_round_trip():
    from unirl_b200.models.sd3.hf_keys import from_diffusers, to_diffusers

    pipe = _pipe("tiny-sd3")
    m = pipe.bundle.transformer
    h = m.cfg.hidden_size
    native = {k: v.detach().clone() for k, v in m.state_dict().items()}
    split = to_diffusers(native, m.cfg.num_joint_blocks, h)
    assert f"transformer_blocks.0.attn.to_q.weight" in split and split["transformer_blocks.0.attn.to_k.weight"].shape == (h, h)
    assert torch.equal(torch.cat([split[f"transformer_blocks.1.attn.add_{n}_proj.weight"] for n in "qkv"]), native["joint_blocks.1.txt_attn.qkv.weight"])
    hf = dict(split)
    hf.update({"pos_embed.proj.weight": native["patch_embed.weight"].view(h, 4, 2, 2), "pos_embed.proj.bias": native["patch_embed.bias"]})
    back = from_diffusers(hf, m.cfg.num_joint_blocks, m.cfg.dual_attention_blocks)
    assert torch.equal(back["joint_blocks.0.img_attn.qkv.weight"], native["joint_blocks.0.img_attn.qkv.weight"])
    assert torch.equal(back["joint_blocks.0.img_attn2.qkv.bias"], native["joint_blocks.0.img_attn2.qkv.bias"])
    assert back["patch_embed.weight"].shape == native["patch_embed.weight"].shape


def _trainer(overrides):
    cfg = compose("diffusion/tiny_sd3_flowgrpo_cpu", overrides=overrides)
    return DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                            rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                            data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=None)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("algo", ["flowgrpo", "flowdppo", "nft"])
def test_diffusion_training_loop(algo):
    ov = []
    if algo == "flowdppo":
        ov = ["algorithm._target_=unirl_b200.algorithms.flowdppo.FlowDPPO", "~algorithm.clip_range", "~algorithm.old_logp_source"]
    elif algo == "nft":
        ov = ["algorithm._target_=unirl_b200.algorithms.diffusionnft.DiffusionNFT", "~algorithm.clip_range", "~algorithm.old_logp_source",
              "+backend.ema_lora_cfg={rank: 4, alpha: 8, target_modules: [to_q, to_k, to_v, to_out.0]}"]
    tr = _trainer(ov)
    try:
        before = tr.backend.compute_local_param_checksums()[0]
        tr.train(num_rollouts=2)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2 and all("train/policy_loss" in r for r in rows)
        assert tr.backend.compute_local_param_checksums()[0] != before
        if algo == "flowgrpo":
            assert abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4  # first update is on-policy: replay reproduces the rollout log-probs
    finally:
        tr.shutdown()


@pytest.mark.timeout(600)
def test_native_diffusion_engine_own_weights_and_tensor_sync():
    """The native engine keeps its own copy of the transformer; weights arrive by in-memory tensor sync and are fingerprinted."""
    ov = ["rollout._target_=unirl_b200.rollout.engine.native_diffusion.engine.NativeDiffusionRolloutEngine", "~rollout.stage_attrs",
          "+rollout.config={pipeline_cls: unirl_b200.models.sd3.pipeline.SD3Pipeline, pipeline_config_cls: unirl_b200.models.sd3.config.SD3PipelineConfig, "
          "pretrained_model_ckpt_path: 'random:tiny-sd3', model_precision: fp32, autocast_precision: fp32, device: cpu, share_trainer_weights: false}",
          "+sync={_target_: unirl_b200.distributed.weight_sync.full.tensor.TensorWeightSync}"]
    tr = _trainer(ov)
    try:
        assert tr.rollout.compute_local_param_checksums()[0] == tr.backend.compute_local_param_checksums()[0], "engine starts from the trainer's weights"
        tr.train(num_rollouts=2, weight_sync_interval=1)
        assert tr.rollout.compute_local_param_checksums()[0] != tr.backend.compute_local_param_checksums()[0], "trainer moved on after the last update"
        tr._sync_weights()
        assert tr.rollout.compute_local_param_checksums()[0] == tr.backend.compute_local_param_checksums()[0]
        tr.rollout.sleep()
        assert tr.rollout.get_weight_version()[0] >= 2
        tr.rollout.wake_up()
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4
    finally:
        tr.shutdown()


@pytest.mark.timeout(600)
def test_secondary_benchmark_script_runs_on_cpu():
    """``bench_diffusion.py`` (the Flow-DPPO samples/s benchmark) with the tiny preset: one JSON line with the agreed keys."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bench_diffusion.py"), "--device", "cpu", "--preset", "tiny-sd3", "--prompts-per-gpu", "1",
           "--samples-per-prompt", "4", "--micro-batch", "4", "--resolution", "64", "--inference-steps", "4", "--train-timesteps", "2", "--text-len", "7",
           "--steps", "1", "--warmup", "1", "reward.backend.in_channels=4", "+reward.backend.width=8", "backend.fsdp_cfg.activation_checkpointing=false",
           "backend.lora_cfg.rank=4", "backend.lora_cfg.alpha=8", "rollout.config.forward_batch_size=2"]  # the sampler engine runs the 4 samples as two calls
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=500, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    row = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert row["metric"] == "flowdppo_samples_per_s" and row["value"] > 0 and row["config"]["samples_per_prompt"] == 4 and row["steps"] == 1
    assert row["config"]["trained_timesteps"] == 2 and row["config"]["text_tokens"] == 7 and row["e2e"]["h2d_bytes_per_step"] > 0 and row["lora_sync_ms"] > 0


def test_family_specific_stages_z_image_hunyuan_video_and_hunyuan_video15():
    """Behaviour the three families add to the generic core: Z-Image's reversed time / negated output / ``cond + g (cond - uncond)``
    guidance; HunyuanVideo's single guided pass and cropped prompt template; HunyuanVideo-1.5's channel packing of the transformer input."""
    from unirl_b200.models.dit.diffusion import DiTDiffusionParams
    from unirl_b200.models.hunyuan_video import HunyuanVideoPipeline, HunyuanVideoPipelineConfig
    from unirl_b200.models.hunyuan_video.pipeline import PROMPT_PREFIX
    from unirl_b200.models.hunyuan_video15 import HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig
    from unirl_b200.models.z_image import ZImagePipeline, ZImagePipelineConfig
    from unirl_b200.models.dit.conditions import DiTConditions

    kw = dict(model_precision="fp32", autocast_precision="fp32", device="cpu")
    # ---- Z-Image
    z = ZImagePipeline.from_config(ZImagePipelineConfig(pretrained_model_ckpt_path="random:tiny-z-image", **kw))
    cond = DiTConditions(text=z.text_embed.embed(["a red cube", "a tree"]), negative_text=z.text_embed.embed(["", ""]))
    x, sig = torch.randn(2, *z.latent_shape(DiffusionSamplingParams(height=64, width=64))), torch.tensor([0.3])
    p = DiTDiffusionParams(guidance_scale=0.5)
    vc, vu = z.diffusion._branches(x, sig, cond, p)
    model = z.bundle.transformer
    want = -model(x, (1 - sig).expand(2) * 1000.0, cond.text.embeds, None, cond.text.attn_mask).float()
    torch.testing.assert_close(vc, want, rtol=1e-4, atol=1e-5)
    assert vu is not None, "guidance is on for any positive scale"
    torch.testing.assert_close(z.diffusion._velocity(x, sig, cond, p), vc + 0.5 * (vc - vu))
    assert z.diffusion._branches(x, sig, cond, DiTDiffusionParams(guidance_scale=0.0))[1] is None
    # ---- HunyuanVideo: one pass whatever the guidance scale; the template prefix is not part of the conditioning sequence
    hv = HunyuanVideoPipeline.from_config(HunyuanVideoPipelineConfig(pretrained_model_ckpt_path="random:tiny-hunyuan-video", max_sequence_length=300, **kw))
    emb = hv.text_embed.embed(["a dog runs", "a dog runs", "night city"])
    tok = hv.bundle.tokenizers[0]
    longest = max(len(tok.encode(s + "<|eot_id|>")) for s in ("a dog runs", "night city")) + 1
    assert emb.embeds.shape[1] == min(longest, hv.bundle.text_encoders[0].cfg.max_length) < len(tok.encode(PROMPT_PREFIX)), "the template prefix is cropped off"
    assert torch.equal(emb.embeds[0], emb.embeds[1]) and emb.pooled is not None
    hcond = DiTConditions(text=emb, negative_text=emb)
    xv = torch.randn(3, *hv.latent_shape(DiffusionSamplingParams(height=32, width=32, num_frames=5)))
    v, none = hv.diffusion._branches(xv, torch.tensor([0.7]), hcond, DiTDiffusionParams(guidance_scale=6.0))
    assert none is None and v.shape == xv.shape
    v2, _ = hv.diffusion._branches(xv, torch.tensor([0.7]), hcond, DiTDiffusionParams(guidance_scale=1.0))
    assert not torch.allclose(v, v2), "the guidance scale enters through its embedding"
    # ---- HunyuanVideo-1.5: latents keep the output width; the transformer sees latents + conditioning latents + mask
    h15 = HunyuanVideo15Pipeline.from_config(HunyuanVideo15PipelineConfig(pretrained_model_ckpt_path="random:tiny-hunyuan-video15", **kw))
    shape = h15.latent_shape(DiffusionSamplingParams(height=32, width=32, num_frames=5))
    t15 = h15.bundle.transformer.cfg
    assert shape[0] == t15.out_channels == 4 and t15.in_channels == 9
    x15 = torch.randn(2, *shape)
    c15 = DiTConditions(text=h15.text_embed.embed(["a", "b"]))
    packed = h15.diffusion._model_input(x15, c15)
    assert packed.shape[1] == 9 and torch.equal(packed[:, :4], x15) and float(packed[:, 4:].abs().sum()) == 0.0
    assert h15.diffusion._velocity(x15, torch.tensor([0.5]), c15, DiTDiffusionParams(guidance_scale=1.0)).shape == x15.shape


def test_qwen_image_text_stage_with_a_language_model_tower():
    """Qwen-Image's conditioning: chat template, decoder-only language model (the package's own decoder behind the encoder interface),
    system prefix cut off, zero rows and a mask at the padding, no pooled vector, identical prompts encoded once."""
    from unirl_b200.models.dit.llm_tower import LLMTextTower
    from unirl_b200.models.qwen3.modeling import Qwen3Config
    from unirl_b200.models.qwen_image import QwenImagePipeline, QwenImagePipelineConfig
    from unirl_b200.models.qwen_image.pipeline import PROMPT_PREFIX, PROMPT_SUFFIX, QwenImageTextEmbedStage

    pipe = QwenImagePipeline.from_config(QwenImagePipelineConfig(pretrained_model_ckpt_path="random:tiny-qwen-image", model_precision="fp32", autocast_precision="fp32",
                                                                 device="cpu", max_sequence_length=64))
    assert isinstance(pipe.text_embed, QwenImageTextEmbedStage)
    tok = pipe.bundle.tokenizers[0]
    tdim = pipe.bundle.spec.transformer.text_dim
    tower = LLMTextTower(Qwen3Config.tiny(vocab_size=512, hidden_size=tdim, head_dim=16, attention_bias=True, qk_norm=False), dtype=torch.float32).init_weights(3)
    stage = QwenImageTextEmbedStage([tower], [tok], "single", tdim, 64)
    prompts = ["a red cube on a table", "a tree", "a red cube on a table"]
    emb = stage.embed(prompts)
    crop = len(tok.encode(PROMPT_PREFIX))
    lens = [len(tok.encode(PROMPT_PREFIX + s + PROMPT_SUFFIX)) - crop for s in prompts]
    assert emb.pooled is None and emb.embeds.shape == (3, max(lens), tdim) and emb.attn_mask.sum(1).tolist() == lens
    assert torch.equal(emb.embeds[0], emb.embeds[2])
    assert float(emb.embeds[1, lens[1]:].abs().max()) == 0.0 and float(emb.embeds[1, : lens[1]].abs().min(0).values.max()) > 0.0
    # the kept rows are the tower's hidden states of the templated prompt from the end of the prefix on (causal: padding cannot reach them)
    ids = torch.tensor([[int(i) % 512 for i in tok.encode(PROMPT_PREFIX + "a tree" + PROMPT_SUFFIX)]])
    full, _ = tower(ids, torch.ones_like(ids))
    torch.testing.assert_close(emb.embeds[1, : lens[1]], full[0, crop:], rtol=1e-4, atol=1e-5)
    # the pipeline's own stage (stand-in tower of the random preset) follows the same contract
    e2 = pipe.text_embed.embed(prompts)
    assert e2.embeds.shape[:2] == emb.embeds.shape[:2] and e2.pooled is None


@pytest.mark.timeout(600)
def test_engine_with_its_own_pipeline_samples_with_the_strategy_named_on_the_trainers_pipeline():
    """``pipeline.strategy`` names a step strategy other than the family's default; the sampler engine has a pipeline of its own.  The
    engine's emitted log-probs are the PPO anchor (``old_logp_source: rollout``), so the first update is on-policy only if the engine
    sampled with the same strategy the trainer replays with."""
    ov = ["rollout._target_=unirl_b200.rollout.engine.native_diffusion.engine.NativeDiffusionRolloutEngine", "~rollout.stage_attrs",
          "+rollout.config={pipeline_cls: unirl_b200.models.sd3.pipeline.SD3Pipeline, pipeline_config_cls: unirl_b200.models.sd3.config.SD3PipelineConfig, "
          "pretrained_model_ckpt_path: 'random:tiny-sd3', model_precision: fp32, autocast_precision: fp32, device: cpu, share_trainer_weights: false}",
          "+sync={_target_: unirl_b200.distributed.weight_sync.full.tensor.TensorWeightSync}", "pipeline._target_=unirl_b200.models.sd3.pipeline.SD3Pipeline",
          "+pipeline.strategy={_target_: unirl_b200.sde.kernels.FlowSDEStrategy}", "algorithm.old_logp_source=rollout"]
    tr = _trainer(ov)
    try:
        assert tr._strategy_name in ("flow", "sde")
        tr.train(num_rollouts=1, weight_sync_interval=1)
        row = [r for r in tr.wandb_logger.history if "train/step" in r][0]
        assert abs(row["train/ratio_mean"] - 1.0) < 1e-4, row["train/ratio_mean"]
    finally:
        tr.shutdown()


def test_image_to_video_request_carries_its_condition_images_into_rollout_and_replay():
    """WAN image-to-video: ``primitives["image"]`` (one picture per sample) becomes the mask + first-frame latents beside the noisy
    latents; the track keeps that condition, replay with it reproduces the rollout, and another picture gives another sample."""
    from unirl_b200.models.wan21.pipeline import Wan21Pipeline, Wan21PipelineConfig
    from unirl_b200.types.primitives import Images

    pipe = Wan21Pipeline.from_config(Wan21PipelineConfig(pretrained_model_ckpt_path="random:tiny-wan", model_precision="fp32", autocast_precision="fp32", device="cpu",
                                                         image_to_video=True))
    req = _req(num_frames=9)
    g = torch.Generator().manual_seed(4)
    pics = torch.rand(3, 3, 48, 80, generator=g)  # another size than the request's: resized to height x width
    req.primitives["image"] = Images(pixels=pics)
    tr = pipe.generate(req).tracks["diffusion"]
    c = pipe.latent_shape(req.sampling_params)[0]
    img = tr.conditions["image"].latents
    assert img.shape == (3, 4 + c, 3, 8, 8) and bool((img[:, :4, 0] == 1).all()) and bool((img[:, :4, 1:] == 0).all())
    assert float((img[0, 4:, 0] - img[2, 4:, 0]).abs().max()) > 1e-4
    tokens = tr.conditions["image_embed"].embeds  # the image encoder's tokens, read by every block's cross-attention
    assert tokens.shape == (3, pipe.bundle.image_encoder.cfg.num_tokens, pipe.bundle.model_config.image_dim) and pipe.bundle.model_config.image_dim > 0
    seg = tr.segment
    out = pipe.diffusion.replay(DiTConditions.from_dict(tr.conditions), segment=seg, params=DiTDiffusionParams(guidance_scale=3.0, true_cfg=True))
    assert float((out.log_probs.detach() - seg.sde_logp).abs().max()) < 1e-5
    req2 = _req(num_frames=9)
    req2.primitives["image"] = Images(pixels=pics.flip(0))
    other = pipe.generate(req2).tracks["diffusion"].segment
    assert float((other.latents[:, -1] - seg.latents[:, -1]).abs().max()) > 1e-4
