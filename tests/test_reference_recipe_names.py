"""Recipes written for the reference: their target names resolve here, and a recipe spelled their way runs."""
import os

import pytest

from unirl_b200.config.instantiate import get_method
from unirl_b200.config.loader import compose

# public names recipes of the reference use as ``_target_`` (model families, engines, reward backends and their specs, transports)
NAMES = [
    "unirl.models.sd3.bundle.SD3Bundle.from_config", "unirl.models.sd3.pipeline.SD3Pipeline", "unirl.models.sd3.conditions.SD3Conditions",
    "unirl.models.wan21.bundle.WAN21Bundle.from_config", "unirl.models.wan21.config.WAN21PipelineConfig", "unirl.models.wan21.pipeline.WAN21Pipeline",
    "unirl.models.wan22.bundle.WAN22Bundle.from_config", "unirl.models.wan22.config.WAN22PipelineConfig", "unirl.models.wan22.pipeline.WAN22Pipeline",
    "unirl.models.qwen_image.bundle.QwenImageBundle.from_config", "unirl.models.qwen_image.config.QwenImagePipelineConfig",
    "unirl.models.flux2_klein.bundle.Flux2KleinBundle.from_config", "unirl.models.flux2_klein.config.Flux2KleinPipelineConfig",
    "unirl.models.z_image.bundle.ZImageBundle.from_config", "unirl.models.z_image.config.ZImagePipelineConfig",
    "unirl.models.hunyuan_video.bundle.HunyuanVideoBundle.from_config", "unirl.models.hunyuan_video.config.HunyuanVideoPipelineConfig",
    "unirl.models.hunyuan_video15.bundle.HunyuanVideo15Bundle.from_config", "unirl.models.hunyuan_video15.config.HunyuanVideo15PipelineConfig",
    "unirl.models.hunyuan_image3.bundle.HunyuanImage3Bundle.from_meta_config", "unirl.models.hunyuan_image3.config.HunyuanImage3PipelineConfig",
    "unirl.models.hunyuan_image3.pipeline.HunyuanImage3Pipeline.from_bundle",
    "unirl.models.bagel.bundle.BagelBundle.from_config", "unirl.models.bagel.config.BagelPipelineConfig", "unirl.models.bagel.pipeline.BagelPipeline",
    "unirl.models.bagel.diffusion.BagelDiffusionParams",
    "unirl.models.qwen3.bundle.Qwen3Bundle.from_config", "unirl.models.qwen3.pipeline.Qwen3Pipeline.from_bundle", "unirl.models.qwen_vl.bundle.QwenVLBundle.from_config",
    "unirl.rollout.engine.sglang_llm.engine.SGLangLLMRolloutEngine", "unirl.rollout.engine.sglang_llm.config.SGLangLLMEngineConfig",
    "unirl.rollout.engine.sglang.engine.SGLangRolloutEngine", "unirl.rollout.engine.sglang.config.SGLangEngineConfig",
    "unirl.rollout.engine.vllm_omni.engine.VLLMOmniRolloutEngine", "unirl.rollout.engine.vllm_omni.config.VLLMOmniEngineConfig",
    "unirl.rollout.engine.composed.engine.ComposedRolloutEngine", "unirl.rollout.engine.composed.config.ComposedRolloutEngineConfig",
    "unirl.rollout.engine.trainside.engine.TrainsideRolloutEngine",
    "unirl.reward.service.RewardService", "unirl.reward.remote.RemoteRewardBackend", "unirl.reward.remote.RemoteRewardSpec",
    "unirl.reward.local.clip.ClipRewardScorer", "unirl.reward.local.clip.ClipSpec", "unirl.reward.local.pickscore.PickScoreRewardScorer",
    "unirl.reward.local.pickscore.PickScoreSpec", "unirl.reward.local.hpsv2.HPSv2RewardScorer", "unirl.reward.local.hpsv2.HPSv2Spec",
    "unirl.reward.local.hpsv3.HPSv3RewardScorer", "unirl.reward.local.image_reward.ImageRewardScorer", "unirl.reward.local.aesthetic.AestheticRewardScorer",
    "unirl.reward.local.ocr.OCRRewardScorer", "unirl.reward.local.ocr.OCRSpec", "unirl.reward.local.geneval2.GenEval2RewardScorer", "unirl.reward.local.geneval2.GenEval2Spec",
    "unirl.reward.local.video.VideoRewardScorer", "unirl.reward.local.video.VideoSpec", "unirl.reward.local.video_pickscore.VideoPickScoreScorer",
    "unirl.reward.local.video_pickscore.VideoPickScoreSpec", "unirl.reward.local.mc_exact_match.MCExactMatchRewardScorer", "unirl.reward.local.mc_exact_match.MCExactMatchSpec",
    "unirl.reward.local.math_boxed.MathBoxedRewardScorer", "unirl.reward.local.mathverify.MathVerifyRewardScorer", "unirl.reward.local.gsm8k_exact_match.GSM8KExactMatchRewardScorer",
    "unirl.distributed.tensor.backend.transfer_queue.simple.SimpleBackend", "unirl.distributed.tensor.backend.transfer_queue.mooncake.MooncakeBackend",
    "unirl.distributed.tensor.backend.transfer_queue.mooncake.MooncakeZeroCopyConfig",
    "unirl.algorithms.grpo.GRPO", "unirl.algorithms.drpo.DRPO", "unirl.algorithms.flowgrpo.FlowGRPO", "unirl.algorithms.flowdppo.FlowDPPO", "unirl.algorithms.diffusionnft.DiffusionNFT",
    "unirl.sde.kernels.FlowSDEStrategy", "unirl.utils.scheduler_utils.AllSDEScheduler", "unirl.types.sampling.DiffusionSamplingParams", "unirl.types.sampling.ARSamplingParams",
    "unirl.train.backend.fsdp.FSDPBackend", "unirl.train.configs.FSDPConfig", "unirl.train.configs.LoraConfig", "unirl.train.backend.base.OptimizerConfig",
    "unirl.train.stack.TrainStack", "unirl.data.data_source.MultimodalRLDataSource", "unirl.distributed.weight_sync.lora.LocalLoraWeightSync", "hydra.utils.get_class",
]


def test_every_public_target_name_resolves():
    missing = []
    for n in NAMES:
        try:
            assert get_method(n) is not None
        except Exception as e:  # noqa: BLE001
            missing.append(f"{n}: {type(e).__name__}: {e}")
    assert not missing, "\n".join(missing)


def test_engine_configurations_translate():
    from unirl_b200.rollout.engine.compat import SGLangEngineConfig, SGLangLLMEngineConfig, VLLMOmniEngineConfig

    ar = SGLangLLMEngineConfig(pretrained_model_ckpt_path="random:tiny", tp_size=2, max_new_tokens=64, temperature=1.0, top_p=1.0, top_k=0, samples_pre_expanded=True,
                               chat_template_kwargs={"enable_thinking": True}, engine_kwargs={"mem_fraction_static": 0.3, "disable_cuda_graph": True, "cuda_graph_max_bs": 16},
                               host="10.0.0.1", port=30000).to_native()
    assert ar.tp_size == 2 and ar.max_new_tokens == 64 and ar.samples_pre_expanded and not ar.use_cuda_graph and ar.max_running_requests == 16
    d = SGLangEngineConfig(model_family="wan21", forward_batch_size=4, tp_size=2, engine_kwargs={"model_path": "random:tiny-wan"}).to_native()
    assert d.pipeline_cls.endswith("Wan21Pipeline") and d.forward_batch_size == 4 and d.tp_size == 2 and d.pretrained_model_ckpt_path == "random:tiny-wan"
    v = VLLMOmniEngineConfig(model_path="", model_family="qwen_image", omni_extra={"tensor_parallel_size": 4}).to_native()
    assert v.pipeline_cls.endswith("QwenImagePipeline") and v.tp_size == 4 and v.pretrained_model_ckpt_path == "random:qwen-image"
    with pytest.raises(ValueError):
        SGLangEngineConfig(model_family="unknown").to_native()


@pytest.mark.timeout(600)
def test_a_recipe_spelled_the_reference_way_runs(tmp_path, monkeypatch):
    from unirl_b200.trainer.diffusion import DiffusionTrainer

    prompts = tmp_path / "prompts.txt"
    prompts.write_text("a red cube\na tree at dusk\ntwo dogs\na bowl of ramen\n")
    monkeypatch.setenv("DATA_PATH", str(prompts))
    cfg = compose("compat/sd3_flowdppo_reference_names_cpu")
    assert cfg.sampling.scheduler.num_timesteps == 6 and cfg.algorithm.params.scheduler.num_timesteps == 6  # relative reference, also through ${sampling}
    tr = DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                          reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                          sync_cfg=cfg.get("sync"), logging_cfg=None)
    try:
        before = tr.backend.compute_local_param_checksums()[0]
        tr.train(num_rollouts=1)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert rows and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4 and "train/kl_mask_fraction" in rows[0]
        assert tr.backend.compute_local_param_checksums()[0] != before
    finally:
        tr.shutdown()


@pytest.mark.timeout(600)
def test_a_language_model_recipe_spelled_the_reference_way_runs(tmp_path, monkeypatch):
    import json

    from unirl_b200.rollout.engine.compat import SGLangLLMRolloutEngine
    from unirl_b200.trainer.ar import ARTrainer

    data = tmp_path / "math.jsonl"
    data.write_text("".join(json.dumps({"prompt": f"What is {i}+{i}? Put the answer in \\boxed{{}}.", "metadata": {"answer": str(2 * i)}}) + "\n" for i in range(8)))
    monkeypatch.setenv("DATA_PATH", str(data))
    cfg = compose("compat/qwen3_grpo_reference_names_cpu")
    assert cfg.data_source.args.run.eval_data_path == str(data)  # a default that is itself an environment reference
    tr = ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                   reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                   sync_cfg=cfg.get("sync"), logging_cfg=None)
    try:
        assert isinstance(tr.pool.local_role(tr.rollout), SGLangLLMRolloutEngine)
        tr.train(num_rollouts=1)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert rows and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4
    finally:
        tr.shutdown()
