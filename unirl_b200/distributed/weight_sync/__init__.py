"""Trainer → rollout weight synchronisation (full weights and LoRA adapters)."""
