"""Vision-language policy: 3-axis rotary positions, rollout/replay alignment with images, and the GRPO loop."""
import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.models.qwen_vl import QwenVLARConditions, QwenVLConfig, QwenVLPipeline, QwenVLPipelineConfig
from unirl_b200.models.qwen_vl.modeling import mrope_positions
from unirl_b200.trainer.ar import ARTrainer
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.sampling import ARSamplingParams


def test_mrope_positions_text_image_text():
    cfg = QwenVLConfig.tiny()
    toks = torch.tensor([7, 8, cfg.vision_start_token_id] + [cfg.image_token_id] * 4 + [9, 10])
    pos, delta = mrope_positions(toks, [(1, 4, 4)], cfg)  # 4x4 patches merge 2x2 -> a 2x2 grid of placeholder tokens
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    assert pos[:, 3:7].tolist() == [[3, 3, 3, 3], [3, 3, 4, 4], [3, 4, 3, 4]]
    assert pos[:, 7:].tolist() == [[5, 6]] * 3 and delta == 7 - 9
    text_only, d0 = mrope_positions(torch.tensor([1, 2, 3]), [], cfg)
    assert text_only.tolist() == [[0, 1, 2]] * 3 and d0 == 0


def test_rollout_and_replay_agree_with_images():
    pipe = QwenVLPipeline.from_config(QwenVLPipelineConfig(pretrained_model_ckpt_path="random:tiny-vl", model_precision="fp32", device="cpu", min_pixels=64,
                                                            max_pixels=1024))
    req = RolloutReq(sample_ids=["a/0", "a/1", "b/0"], group_ids=["a", "a", "b"],
                     primitives={"text": Texts.from_list(["what is this", "what is this", "and this one"]), "image": Images(pixels=torch.rand(3, 3, 20, 28))},
                     sampling_params=ARSamplingParams(max_new_tokens=6, temperature=1.0, top_p=1.0, top_k=0))
    tr = pipe.generate(req).tracks["ar"]
    conds = QwenVLARConditions.from_dict(tr.conditions)
    assert len(conds.pixel_values) == 3 and conds.image_grid_thw[0].tolist() == [[1, 4, 8]]
    lp = pipe.ar.replay(conds, segment=tr.segment, temperature=1.0)
    assert float((lp.detach() - tr.segment.log_probs).abs().max()) < 1e-4
    part = conds.slice(1, 3)  # the image lists travel with the prompt rows
    assert len(part.pixel_values) == 2 and torch.equal(part.pixel_values[0], conds.pixel_values[1])
    # a policy may SAMPLE the placeholder id: in the response it is an ordinary token (the decode step embedded it as text), so the replay
    # of a response that contains it must neither look for a vision feature nor move the positions of what follows
    seg = tr.segment
    forced = seg.tokens.clone()
    forced[1] = pipe.ar.model.transformer.cfg.image_token_id
    original, seg.tokens = seg.tokens, forced
    try:
        lp2 = pipe.ar.replay(conds, segment=seg, temperature=1.0)
    finally:
        seg.tokens = original
    assert lp2.shape == lp.shape and torch.isfinite(lp2).all()
    assert float((lp2[0] - lp[0]).abs()) < 1e-5  # the token before the forced one sees the same context


@pytest.mark.timeout(600)
def test_vl_grpo_loop():
    cfg = compose("ar/tiny_qwen_vl_grpo_cpu", overrides=[])
    tr = ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                   reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                   logging_cfg=None)
    try:
        tr.train(num_rollouts=2)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2 and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-3
    finally:
        tr.shutdown()


def _vl_trainer(overrides):
    cfg = compose("ar/tiny_qwen_vl_grpo_cpu", overrides=overrides)
    return ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                     reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                     sync_cfg=cfg.get("sync"), logging_cfg=None)


_ENGINE = ["rollout._target_=unirl_b200.rollout.engine.native_ar.engine.NativeARRolloutEngine", "~rollout.stage_attrs",
           "+rollout.config={pretrained_model_ckpt_path: 'random:tiny-vl', model_precision: fp32, max_new_tokens: 8, detokenize: false, max_running_requests: 16}"]


@pytest.mark.timeout(600)
def test_vl_grpo_with_the_rollout_engine_sharing_the_trainers_weights():
    """The dedicated rollout engine serves a vision-language policy: image preprocessing and the multimodal prefill run inside the engine,
    on the trainer's replica when both share a device."""
    tr = _vl_trainer(_ENGINE)
    try:
        tr.train(num_rollouts=2)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2 and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-3 and abs(rows[1]["train/ratio_mean"] - 1.0) < 1e-3
    finally:
        tr.shutdown()


@pytest.mark.timeout(900)
def test_vl_grpo_with_a_tensor_parallel_rollout_engine_over_gloo():
    """Two workers: a data-parallel trainer and ONE tensor-parallel engine (decoder sharded over both ranks, vision tower whole on each)
    with weights of its own, refreshed from the trainer's full tensors every step; the replay reproduces the engine's log-probs."""
    ov = _ENGINE[:2] + ["+rollout.config={pretrained_model_ckpt_path: 'random:tiny-vl', model_precision: fp32, max_new_tokens: 8, detokenize: false, "
                        "max_running_requests: 16, tp_size: 2, share_trainer_weights: false, tp_collectives: nccl}",
                        "num_devices=2", "pool_backend=mp", "+rollout_parallel={tp: 2}", "batch_size=4",
                        "+sync={_target_: unirl_b200.distributed.weight_sync.full.tensor.TensorWeightSync}"]
    tr = _vl_trainer(ov)
    try:
        tr.train(num_rollouts=2, weight_sync_interval=1)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 2 and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-3 and abs(rows[1]["train/ratio_mean"] - 1.0) < 1e-3
        assert rows[1]["train/rollout_replay_logp_absdiff_max"] < 1e-3
    finally:
        tr.shutdown()
