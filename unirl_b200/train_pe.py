"""Prompt-enhancement training entry point: ``python -m unirl_b200.train_pe --config-name=pe/<recipe> [key=value …]``.
Parity: ``unirl/train_pe.py:21-38``."""

from __future__ import annotations

from unirl_b200.config.loader import main_entry
from unirl_b200.trainer.pe import PETrainer


@main_entry(default_config="pe/tiny_pe_cpu")
def main(cfg) -> None:
    trainer = PETrainer(cfg=cfg, batch_size=cfg.batch_size, ar_cfg=cfg.ar, diffusion_cfg=cfg.diffusion, reward_cfg=cfg.reward, data_source_cfg=cfg.data_source,
                        sampling_cfg=cfg.sampling, composed_cfg=cfg.get("composed"), logging_cfg=cfg.get("logging"),
                        reward_propagation=str(cfg.get("reward_propagation", "mean")))
    try:
        trainer.train(num_rollouts=int(cfg.get("num_rollouts", 100)))
    finally:
        trainer.shutdown()


if __name__ == "__main__":
    main()
