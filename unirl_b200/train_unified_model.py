"""Unified-model training entry point: ``python -m unirl_b200.train_unified_model --config-name=unified_model/<recipe> [key=value …]``.
Parity: ``unirl/train_unified_model.py:23-50``."""

from __future__ import annotations

from unirl_b200.config.loader import main_entry
from unirl_b200.trainer.unified_model import UnifiedModelTrainer


@main_entry(default_config="unified_model/tiny_unified_t2i_cpu")
def main(cfg) -> None:
    trainer = UnifiedModelTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                                  rollout_cfg=cfg.get("rollout"), ar_rollout_cfg=cfg.get("ar_rollout"), dit_rollout_cfg=cfg.get("dit_rollout"),
                                  enable_fsdp_offload=bool(cfg.get("enable_fsdp_offload", False)), devices_per_replica=cfg.get("devices_per_replica"),
                                  reward_cfg=cfg.reward, ar_algorithm_cfg=cfg.get("ar_algorithm") or (cfg.get("algorithm") or {}).get("ar"),
                                  image_algorithm_cfg=cfg.get("image_algorithm") or (cfg.get("algorithm") or {}).get("image"), stack_cfg=cfg.stack,
                                  data_source_cfg=cfg.data_source,
                                  sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=cfg.get("logging"), mode=str(cfg.get("mode", "t2i")),
                                  rollout_dump_dir=cfg.get("rollout_dump_dir") or cfg.get("dump_dir"))
    try:
        trainer.train(num_rollouts=int(cfg.get("num_rollouts", 100)), weight_sync_interval=int(cfg.get("weight_sync_interval", 1)),
                      save_interval=int(cfg.get("save_interval", 0)), save_dir=cfg.get("save_dir"), load_dir=cfg.get("load_dir"))
    finally:
        trainer.shutdown()


if __name__ == "__main__":
    main()
