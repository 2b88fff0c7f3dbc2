"""Prompt-enhancement composition of an LLM and a diffusion pipeline.  Parity: ``unirl/models/pe/``."""
from unirl_b200.models.pe.pipeline import PEPipeline

__all__ = ["PEPipeline"]
