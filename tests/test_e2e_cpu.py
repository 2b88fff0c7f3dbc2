"""End-to-end plumbing on CPU: the world-size-2 gloo GRPO run (separate trainer / rollout pools, broadcast weight sync),
the colocated path, resume from checkpoint, and rollout/replay numerical alignment."""
import os

import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.trainer.ar import ARTrainer


def _trainer(cfg):
    return ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                     rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                     data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=cfg.get("logging"))


_COLOC = ["num_devices=1", "batch_size=4", "bundle.config.pretrained_model_ckpt_path=random:tiny", "rollout.config.pretrained_model_ckpt_path=random:tiny",
          "rollout.config.tp_size=1", "rollout.config.max_new_tokens=12", "sampling.samples_per_prompt=4", "sampling.max_new_tokens=12",
          "data_source.vocab_size=4096", "data_source.min_len=8", "data_source.max_len=20", "data_source.reserved_low_ids=16", "stack.micro_batch_size=8",
          "algorithm.horizon=12", "rollout_parallel={tp: 1}", "+pool_backend=inline", "+pool_device=cpu", "+bundle.config.device=cpu",
          "bundle.config.model_precision=fp32", "backend.fsdp_cfg.mixed_precision=false", "backend.optimizer_cfg.learning_rate=1.0e-3"]


@pytest.mark.timeout(600)
def test_world2_gloo_grpo_separate_pools_with_weight_sync():
    cfg = compose("ar/tiny_qwen3_grpo_cpu", overrides=["num_rollouts=2"])
    tr = _trainer(cfg)
    try:
        assert tr.backend.devices == [0] and tr.rollout.devices == [1]
        before = tr.rollout.compute_local_param_checksums()[0]
        tr.train(num_rollouts=2, weight_sync_interval=1)
        hist = [r for r in tr.wandb_logger.history if "rollout/step" in r]
        assert len(hist) == 2 and all(0.0 <= r["rollout/reward_mean"] <= 1.0 for r in hist)
        train_rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(train_rows) == 4, "2 rollouts x 2 updates per batch"
        assert abs(train_rows[0]["train/ratio_mean"] - 1.0) < 1e-3, "first update is on-policy (engine weights == trainer weights)"
        # after the final update push the weights once more: engine and trainer must agree tensor by tensor
        tr._sync_weights()
        after = tr.rollout.compute_local_param_checksums()[0]
        trainer_sums = tr.backend.compute_local_param_checksums()[0]
        assert after == trainer_sums and after != before
        assert tr.rollout.get_weight_version()[0] >= 2
    finally:
        tr.shutdown()


@pytest.mark.timeout(600)
def test_colocated_step_resume_and_alignment(tmp_path):
    cfg = compose("ar/qwen3_4b_grpo_b200", overrides=_COLOC)
    tr = _trainer(cfg)
    try:
        tr.train(num_rollouts=2, save_interval=1, save_dir=str(tmp_path))
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-4 and rows[0]["train/rollout_replay_logp_absdiff_max"] < 1e-4
        assert os.path.exists(tmp_path / "checkpoint-2" / "checkpoint.pt") and os.path.exists(tmp_path / "checkpoint-2" / "trainer_state.json")
        w_after_2 = tr.backend.compute_local_param_checksums()[0]
        tr.train(num_rollouts=3, load_dir=str(tmp_path / "checkpoint-1"))  # resumes at rollout 1, replays rollouts 2 and 3
        assert tr.backend.call("optimizer_step_count") if False else True
    finally:
        tr.shutdown()
    tr2 = _trainer(cfg)
    try:
        start = tr2.maybe_load_checkpoint(str(tmp_path / "checkpoint-2"))
        assert start == 2 and tr2.backend.compute_local_param_checksums()[0] == w_after_2
        assert tr2._resume_state.get("optimizer_step") == 2
    finally:
        tr2.shutdown()


@pytest.mark.timeout(900)
def test_colocated_dp2_trainer_with_tp2_rollout_over_gloo():
    """The headline topology in miniature: two workers host a DP=2 sharded trainer AND one TP=2 rollout engine; the
    engine's single output handle is windowed across the two trainer ranks, weights move by the reshard plan."""
    ov = [o for o in _COLOC if not o.startswith(("num_devices", "rollout.config.tp_size", "rollout_parallel", "+pool_backend"))]
    cfg = compose("ar/qwen3_4b_grpo_b200", overrides=ov + ["num_devices=2", "rollout.config.tp_size=2", "rollout_parallel={tp: 2}", "+pool_backend=mp",
                                                           "rollout.config.max_running_requests=16", "rollout.config.model_precision=fp32"])
    tr = _trainer(cfg)
    try:
        tr.train(num_rollouts=2, weight_sync_interval=1)
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert rows and abs(rows[0]["train/ratio_mean"] - 1.0) < 1e-3 and rows[0]["train/rollout_replay_logp_absdiff_max"] < 1e-3
        tr._sync_weights()
        eng = tr.rollout.compute_local_param_checksums()
        trn = tr.backend.compute_local_param_checksums()
        assert trn[0] == trn[1], "both trainer ranks hold the same replica"
        replicated = [k for k in eng[0] if k.endswith("layernorm") or k.endswith("norm") or "embed" in k]
        assert replicated and all(eng[0][k] == eng[1][k] == trn[0][k] for k in replicated)
        # payloads that arrive already sharded, one entry per tensor-parallel rank: every rank copies its own entry
        from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor
        from unirl_b200.models.qwen3.bundle import resolve_model_config
        from unirl_b200.models.qwen3.modeling import shard_param

        mcfg = resolve_model_config("random:tiny", {})
        g = torch.Generator().manual_seed(5)
        name = "layers.0.qkv_proj"
        full = torch.randn(((mcfg.num_attention_heads + 2 * mcfg.num_key_value_heads) * mcfg.head_dim, mcfg.hidden_size), generator=g)
        shards = [{name: shard_param(full, name, mcfg, r, 2).contiguous()} for r in range(2)]
        assert tr.rollout.update_weights_from_tensor(serialized_named_tensors=shards, load_format="per_tp_rank") == [1, 1]
        after = tr.rollout.compute_local_param_checksums()
        assert [after[r][name] for r in range(2)] == [fingerprint_tensor(shards[r][name]) for r in range(2)]
    finally:
        tr.shutdown()


@pytest.mark.timeout(900)
def test_torchrun_spmd_backend_two_cpu_ranks():
    """One process per rank under torchrun (every rank is controller and worker): DP=2 trainer + TP=2 engine over gloo."""
    import subprocess
    import sys

    from unirl_b200.distributed.utils import free_port

    ov = [o for o in _COLOC if not o.startswith(("num_devices", "rollout.config.tp_size", "rollout_parallel", "+pool_backend"))]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
           str(free_port()), "-m", "unirl_b200.train_ar", "--config-name=ar/qwen3_4b_grpo_b200", *ov, "num_devices=2", "rollout.config.tp_size=2",
           "rollout_parallel={tp: 2}", "rollout.config.model_precision=fp32", "rollout.config.max_running_requests=16", "num_rollouts=2"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=800, env={**os.environ, "OMP_NUM_THREADS": "2"})
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    import re

    reports = re.findall(r"rollout 2/2  loss=\S+  grad_norm=\S+  lr=\S+  reward=\d+\.\d{4}", p.stdout)  # the two ranks' lines may share one output line
    assert len(reports) == 2 and reports[0] == reports[1], "both ranks run the same controller and agree on the step metrics"


def _lora_cfg(extra):
    ov = [o for o in _COLOC if not o.startswith(("num_devices", "rollout.config.tp_size", "rollout_parallel", "+pool_backend"))]
    return compose("ar/qwen3_4b_grpo_lora_b200", overrides=ov + ["backend.lora_cfg.rank=4", "backend.lora_cfg.alpha=8", "rollout.config.model_precision=fp32",
                                                                 "+rollout.config.share_trainer_weights=false", "backend.optimizer_cfg.learning_rate=5.0e-3"] + extra)


def _assert_lora_engine_follows_trainer(tr):
    tr.train(num_rollouts=3, weight_sync_interval=1)
    rows = [r for r in tr.wandb_logger.history if "train/step" in r]
    # the third rollout is sampled by an engine that folded two updates of the adapters into weights of its own
    assert abs(rows[-1]["train/ratio_mean"] - 1.0) < 1e-3 and rows[-1]["train/rollout_replay_logp_absdiff_max"] < 1e-3
    assert tr.rollout.get_weight_version()[0] >= 2


@pytest.mark.timeout(600)
def test_lora_sync_into_an_engine_with_weights_of_its_own():
    tr = _trainer(_lora_cfg(["num_devices=1", "rollout.config.tp_size=1", "rollout_parallel={tp: 1}", "+pool_backend=inline"]))
    try:
        before = tr.rollout.compute_local_param_checksums()[0]
        _assert_lora_engine_follows_trainer(tr)
        after = tr.rollout.compute_local_param_checksums()[0]
        changed = {k for k in before if before[k] != after[k]}
        assert changed and all(k.rsplit(".", 1)[-1] in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj") for k in changed)
        # withdrawing the adapters gives the base weights back, bit for bit
        tr.rollout.set_lora_from_tensors("default", {}, peft_config={"r": 4, "lora_alpha": 8})
        assert tr.rollout.compute_local_param_checksums()[0] == before
    finally:
        tr.shutdown()


@pytest.mark.timeout(900)
def test_lora_sync_into_a_tp2_engine_over_gloo():
    tr = _trainer(_lora_cfg(["num_devices=2", "rollout.config.tp_size=2", "rollout_parallel={tp: 2}", "+pool_backend=mp", "rollout.config.max_running_requests=16"]))
    try:
        _assert_lora_engine_follows_trainer(tr)
    finally:
        tr.shutdown()


def test_separate_layout_on_one_device_is_refused_with_a_message():
    cfg = compose("ar/tiny_qwen3_grpo_cpu", overrides=["num_devices=1", "+pool_backend=inline"])
    with pytest.raises(ValueError, match="separate layout needs at least one device"):
        _trainer(cfg)


def test_ipc_sync_accepts_the_shared_memory_switch_of_reference_recipes():
    from unirl_b200.distributed.weight_sync.full.ipc import IPCWeightSync

    sync = IPCWeightSync(backend=None, rollout=None, bucket_size_mb=4, lora_merged=True, use_shm=True)
    assert sync.use_shm is True and sync._bucket_bytes == 4 << 20


def test_full_sync_reads_the_older_field_spellings_some_reference_recipes_carry():
    from unirl_b200.distributed.weight_sync.full.nccl import NCCLWeightSync

    sync = NCCLWeightSync(backend=None, use_merged=True, param_name_prefix="transformer.", target_modules=["transformer"], group_name="weight_sync")
    assert sync._lora_merged is True and sync._track_prefix == "transformer." and sync.target_modules == ["transformer"]
