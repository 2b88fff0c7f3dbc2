"""Diffusion training entry point: ``python -m unirl_b200.train_diffusion --config-name=diffusion/<recipe> [key=value …]``.

Serves every DiT family (SD3, WAN, Qwen-Image, FLUX.2 klein, Z-Image, HunyuanVideo) with FlowGRPO, Flow-DPPO or
DiffusionNFT.  Parity: ``unirl/train_diffusion.py:22-50``.
"""

from __future__ import annotations

from unirl_b200.config.loader import main_entry
from unirl_b200.trainer.diffusion import DiffusionTrainer


@main_entry(default_config="diffusion/tiny_sd3_flowgrpo_cpu")
def main(cfg) -> None:
    trainer = DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                               rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                               data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=cfg.get("logging"),
                               adv_normalization_scope=cfg.get("adv_normalization_scope", "group"),
                               normalize_adv_by_std=bool(cfg.get("normalize_adv_by_std", True)))
    try:
        trainer.train(num_rollouts=int(cfg.get("num_rollouts", 100)), weight_sync_interval=int(cfg.get("weight_sync_interval", 1)),
                      save_interval=int(cfg.get("save_interval", 0)), save_dir=cfg.get("save_dir"), load_dir=cfg.get("load_dir"),
                      save_mode=str(cfg.get("save_mode", "full")))
    finally:
        trainer.shutdown()


if __name__ == "__main__":
    main()
