from unirl_b200.types.conditions.base import Condition, Modality  # noqa: F401
from unirl_b200.types.conditions.fused_multimodal import FusedMultimodalCondition  # noqa: F401
from unirl_b200.types.conditions.image import ImageEmbedCondition, ImageLatentCondition  # noqa: F401
from unirl_b200.types.conditions.text import TextEmbedCondition, TextTokenCondition  # noqa: F401
