"""Device status words reach the host as named exceptions at step boundaries; per-device bookkeeping of kernel attributes."""
import pytest
import torch

from unirl_b200.ops._ext import have_ext


@pytest.mark.skipif(not have_ext(), reason="native extension not built")
def test_per_device_first_use_bookkeeping():
    from unirl_b200.ops._ext import require_ext

    C = require_ext()
    # device 1's first launch must configure its kernels although device 0 was configured before; repeats do not
    assert C.per_device_first_use([0, 0, 1, 0, 1, 7, 7]) == [True, False, True, False, False, True, False]
    assert C.per_device_first_use([-1, -1, 64]) == [True, True, True]  # out-of-range ids never cache


@pytest.mark.gpu
def test_host_written_status_word_raises_at_the_next_boundary():
    """The host writes a code into the status word (no kernel is made to give up); the next boundary check raises and clears it."""
    from unirl_b200.ops._ext import require_ext
    from unirl_b200.ops.status import DeviceKernelError, check_device_status

    C = require_ext()
    check_device_status("test start")
    C.set_gemm_status(103)
    with pytest.raises(DeviceKernelError) as e:
        check_device_status("unit test boundary")
    assert e.value.code == 103 and "unit test boundary" in str(e.value)
    check_device_status("after clear")  # cleared by the failing check


@pytest.mark.gpu
def test_trainer_and_engine_raise_on_a_status_word():
    """optimizer_step and the rollout engine's generate stop on a non-zero word instead of training / returning garbage."""
    from unirl_b200.config.loader import compose
    from unirl_b200.ops._ext import require_ext
    from unirl_b200.ops.status import DeviceKernelError
    from unirl_b200.trainer.ar import ARTrainer

    C = require_ext()
    cfg = compose("ar/qwen3_4b_grpo_b200", overrides=[
        "num_devices=1", "batch_size=2", "bundle.config.pretrained_model_ckpt_path=random:tiny", "rollout.config.pretrained_model_ckpt_path=random:tiny",
        "rollout.config.tp_size=1", "rollout.config.max_new_tokens=8", "sampling.samples_per_prompt=2", "sampling.max_new_tokens=8",
        "data_source.vocab_size=4096", "data_source.min_len=8", "data_source.max_len=16", "data_source.reserved_low_ids=16",
        "stack.micro_batch_size=4", "algorithm.horizon=8", "rollout_parallel={tp: 1}", "+pool_backend=inline"])
    trainer = ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                        rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                        data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"))
    try:
        req = trainer._build_req(trainer.data_source.get_samples(trainer.batch_size), 0)
        trainer.train_step(req, sync_weights=True, rollout_id=0)  # a clean step passes both boundaries
        C.set_gemm_status(122)
        with pytest.raises(Exception) as e:
            trainer.train_step(trainer._build_req(trainer.data_source.get_samples(trainer.batch_size), 1), sync_weights=True, rollout_id=1)
        assert "122" in str(e.value) and ("DeviceKernelError" in str(e.value) or isinstance(e.value, DeviceKernelError))
        assert C.gemm_status(True) == 0
    finally:
        trainer.shutdown()


@pytest.mark.gpu
def test_peer_arena_status_word_is_part_of_the_boundary_check():
    from unirl_b200.ops.status import check_device_status, register_checker

    class FakeArena:
        def __init__(self):
            self.state = torch.zeros(8, dtype=torch.int32, device="cuda")

        def check(self):
            code = int(self.state[4].item())
            if code:
                self.state[4].zero_()
                raise RuntimeError(f"peer wait timed out (code {code})")

    a = FakeArena()
    register_checker(a)
    check_device_status("clean")
    a.state[4] = 315  # written from the host
    with pytest.raises(RuntimeError, match="315"):
        check_device_status("boundary")
    check_device_status("clean again")
