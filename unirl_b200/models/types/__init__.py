"""Model-package contracts: Bundle, Pipeline, stages.  Parity: ``unirl/models/types/*``."""
from unirl_b200.models.types.contracts import (  # noqa: F401
    ARStage,
    ARStep,
    Bundle,
    DecodeStage,
    DiffusionStage,
    DiffusionStep,
    EmbedStage,
    EncodeStage,
    LatentShapeProvider,
    Pipeline,
    ReplayResult,
    left_pad_prompt,
)
