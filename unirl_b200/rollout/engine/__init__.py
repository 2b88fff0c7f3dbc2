"""Rollout engines: in-process trainside engine, native tensor-parallel AR engine, native flow-matching sampler, composed engine."""
from unirl_b200.rollout.engine.base import BaseRolloutEngine, chunked_engine_generate_req  # noqa: F401
