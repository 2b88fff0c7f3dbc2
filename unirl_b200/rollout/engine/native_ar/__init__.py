from unirl_b200.rollout.engine.native_ar.generator import ARGenerator, GenerationOutput  # noqa: F401
from unirl_b200.rollout.engine.native_ar.kv_cache import BlockAllocator, PagedKVCache  # noqa: F401
