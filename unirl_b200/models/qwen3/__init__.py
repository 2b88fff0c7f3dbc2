from unirl_b200.models.qwen3.ar import Qwen3ARStage, Qwen3ARStep  # noqa: F401
from unirl_b200.models.qwen3.bundle import Qwen3Bundle  # noqa: F401
from unirl_b200.models.qwen3.conditions import Qwen3ARConditions  # noqa: F401
from unirl_b200.models.qwen3.config import Qwen3PipelineConfig  # noqa: F401
from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer  # noqa: F401
from unirl_b200.models.qwen3.pipeline import Qwen3Pipeline  # noqa: F401
