"""AR training entry point: ``python -m unirl_b200.train_ar --config-name=ar/<recipe> [key=value …]``.

Thin wrapper around :class:`ARTrainer`; serves pure-LLM (``qwen3``) and vision-language (``qwen_vl``) recipes
under ``examples/ar/``.  Under ``torchrun`` every rank runs this program (spmd pool backend).
Parity: ``unirl/train_ar.py:26-55``.
"""

from __future__ import annotations

from unirl_b200.config.loader import main_entry
from unirl_b200.trainer.ar import ARTrainer


@main_entry(default_config="ar/tiny_qwen3_grpo_cpu")
def main(cfg) -> None:
    trainer = ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                        rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                        data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=cfg.get("logging"),
                        adv_normalization_scope=cfg.get("adv_normalization_scope", "group"),
                        normalize_adv_by_std=bool(cfg.get("normalize_adv_by_std", True)), eval_interval=int(cfg.get("eval_interval", 0)),
                        eval_num_prompts=int(cfg.get("eval_num_prompts", 60)), eval_samples_per_prompt=int(cfg.get("eval_samples_per_prompt", 16)),
                        eval_temperature=float(cfg.get("eval_temperature", 1.0)))
    try:
        trainer.train(num_rollouts=int(cfg.get("num_rollouts", 100)), weight_sync_interval=int(cfg.get("weight_sync_interval", 1)),
                      save_interval=int(cfg.get("save_interval", 0)), save_dir=cfg.get("save_dir"), load_dir=cfg.get("load_dir"),
                      save_mode=str(cfg.get("save_mode", "full")))
    finally:
        trainer.shutdown()


if __name__ == "__main__":
    main()
