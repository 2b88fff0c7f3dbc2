"""FLUX.2 klein on the generic DiT core (double + single stream blocks, empirical-mu schedule).  Parity: ``unirl/models/flux2_klein/``."""
from unirl_b200.models.flux2_klein.pipeline import Flux2KleinBundle, Flux2KleinPipeline, Flux2KleinPipelineConfig
from unirl_b200.models.flux2_klein.schedule import KleinSchedulePolicy

from unirl_b200.models.dit.conditions import DiTConditions as Flux2KleinConditions  # noqa: E402  (the family's conditions record: prompt embeddings, pooled vector, masks, optional negative prompt)

__all__ = ["Flux2KleinConditions", "Flux2KleinBundle", "Flux2KleinPipeline", "Flux2KleinPipelineConfig", "KleinSchedulePolicy"]
