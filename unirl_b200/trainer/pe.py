"""``PETrainer`` — prompt enhancement: an LLM policy rewrites prompts, a diffusion policy renders them, both are trained.

Two complete train stacks (AR: bundle / pipeline / backend / GRPO / stack; diffusion: the same with a flow algorithm) sit
behind one :class:`ComposedRolloutEngine`.  Images are scored; the AR track inherits the mean reward of its children
(``RolloutResp.propagate_rewards``); each track gets its own group-relative advantages and its own optimizer step.
No checkpointing (as in the reference).  Parity: ``unirl/trainer/pe.py:64-145`` (construction), ``:164-272`` (step).
"""

from __future__ import annotations

import logging
import time
from typing import Any, Dict, Tuple

from unirl_b200.config.instantiate import instantiate
from unirl_b200.distributed.group.placement import placement, remote, remote_cfg
from unirl_b200.rollout.engine.composed.engine import ComposedRolloutEngine
from unirl_b200.trainer.base import BaseTrainer
from unirl_b200.trainer.diffusion import _cfg_get
from unirl_b200.types.prompts import RolloutInputs
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import hydrate_if_handle

logger = logging.getLogger(__name__)


class PETrainer(BaseTrainer):
    def __init__(self, *, cfg: Any, batch_size: int, ar_cfg: Any, diffusion_cfg: Any, reward_cfg: Any, data_source_cfg: Any, sampling_cfg: Any,
                 composed_cfg: Any = None, logging_cfg: Any = None, reward_propagation: str = "mean", adv_normalization_scope: str = "group",
                 normalize_adv_by_std: bool = True, pool: Any = None) -> None:
        super().__init__(cfg=cfg, logging_cfg=logging_cfg, pool=pool)
        self.batch_size = int(batch_size)
        self.reward_propagation, self.adv_normalization_scope, self.normalize_adv_by_std = reward_propagation, adv_normalization_scope, bool(normalize_adv_by_std)
        self.data_source = instantiate(data_source_cfg)
        self.sampling_params = instantiate(sampling_cfg)
        # Each policy brings its own rollout engine (``ar.rollout`` / ``diffusion.rollout``).  Recipes written for the reference describe the
        # rollout once at top level instead: a train-side engine over both stages, or a composed engine whose configuration holds the
        # two children's engine configurations; both forms are split into the per-policy engines here.
        top = cfg.get("rollout") if hasattr(cfg, "get") else None
        ar_roll, dit_roll, top_extra = self._split_top_rollout(top)
        with placement(self.pool, fraction=1.0, shared_workers=True):
            self.ar = self._build_side(ar_cfg, ar_roll)
            self.diffusion = self._build_side(diffusion_cfg, dit_roll)
            extra = {**top_extra, **(dict(composed_cfg) if composed_cfg else {})}
            extra.pop("_target_", None)
            self.rollout = remote(ComposedRolloutEngine, ar=self.ar["rollout"], diffusion=self.diffusion["rollout"], **extra)
            self.reward = remote_cfg(reward_cfg)
        from unirl_b200.models.dit.config import resolve_family
        from unirl_b200.models.dit.pipeline import DiTPipeline
        from unirl_b200.sde.runtime import FlowMatchSchedulePolicy

        self._spec = resolve_family(str(_cfg_get(diffusion_cfg, "bundle.config.pretrained_model_ckpt_path", "random:tiny-sd3")))
        t = self._spec.transformer
        self._policy = FlowMatchSchedulePolicy(shift=float(self._spec.shift), use_dynamic_shifting=self._spec.use_dynamic_shifting,
                                               vae_scale_factor=t.vae_scale_factor, patch_size=t.patch_size[-1] * (2 if self._spec.packed_latents else 1))
        self._shape_of = lambda d: DiTPipeline.latent_shape_for(self._spec, d)

    @staticmethod
    def _split_top_rollout(top: Any) -> Tuple[Any, Any, Dict[str, Any]]:
        """A top-level ``rollout`` block → ``(AR engine block, diffusion engine block, options of the composed engine)``."""
        if top is None:
            return None, None, {}
        from unirl_b200.config.aliases import translate
        from unirl_b200.config.node import to_container

        block = to_container(top, resolve=True)
        target = translate(str(block.get("_target_", "")))
        if target.endswith("TrainsideRolloutEngine"):
            rest = {k: v for k, v in block.items() if k not in ("_target_", "stage_attrs")}
            return ({"_target_": target, "stage_attrs": ["ar"], **{k: v for k, v in rest.items() if k != "forward_batch_size"}},
                    {"_target_": target, "stage_attrs": ["diffusion"], **rest}, {})
        if target.endswith("ComposedRolloutEngine"):
            conf = dict(block.get("config") or {})
            children = []
            for key in ("ar", "diffusion"):
                child = dict(conf.get(key) or {})
                if not child:
                    raise ValueError(f"rollout.config.{key}: the composed engine needs its {key} child's engine configuration")
                # ``…sglang_llm.config.SGLangLLMEngineConfig`` names the configuration; the engine class sits beside it as ``…RolloutEngine``
                cfg_target = translate(str(child["_target_"]))
                engine = cfg_target.replace("EngineConfig", "RolloutEngine") if "EngineConfig" in cfg_target else cfg_target
                extra = {"model_config": block["model_config"]} if key == "diffusion" and block.get("model_config") is not None else {}
                children.append({"_target_": engine, "config": child, **extra})
            opts = {k: v for k, v in (("pe_marker", conf.get("pe_marker")), ("ar_system_instruction", conf.get("pe_instruction"))) if v}
            return children[0], children[1], opts
        raise ValueError(f"rollout._target_={target!r}: a prompt-enhancement recipe's top-level rollout is a train-side or a composed engine")

    @staticmethod
    def _build_side(side: Any, rollout_block: Any = None) -> Dict[str, Any]:
        import inspect

        from unirl_b200.config.instantiate import parse_cfg

        bundle = remote_cfg(side.bundle)
        pipeline = remote_cfg(side.pipeline, bundle=bundle)
        backend = remote_cfg(side.backend, bundle=bundle)
        algo_params = inspect.signature(parse_cfg(side.algorithm)["role_cls"]).parameters
        algorithm = remote_cfg(side.algorithm, pipeline=pipeline, **({"backend": backend} if "backend" in algo_params else {}))
        stack = remote_cfg(side.stack, fsdp_backend=backend, algorithm=algorithm)
        rp = parse_cfg(side.rollout if "rollout" in side else rollout_block)
        params = inspect.signature(rp["role_cls"]).parameters
        extra = {"pipeline": pipeline} if "pipeline" in params else ({"bundle": bundle} if "bundle" in params else {})
        rollout = remote(**rp, **extra)
        return {"bundle": bundle, "pipeline": pipeline, "backend": backend, "algorithm": algorithm, "stack": stack, "rollout": rollout}

    def _build_req(self, inputs: RolloutInputs, rollout_id: int) -> RolloutReq:
        sp = self.sampling_params
        d = sp.diffusion
        sigmas = self._policy.compute_sigma(num_inference_steps=int(d.num_inference_steps), height=int(d.height), width=int(d.width))
        return RolloutReq(sample_ids=list(inputs.sample_ids), group_ids=list(inputs.group_ids), primitives=dict(inputs.primitives), sampling_params=sp,
                          sigmas=sigmas, stage_config={"rollout_id": int(rollout_id)}, metadata=list(inputs.metadata) if inputs.metadata else [],
                          init_noise_latent_shape=list(self._shape_of(d)))

    def train_step(self, req: RolloutReq, *, training_progress: float = 0.0, rollout_id: int = 0) -> Tuple[Dict[str, Any], float]:
        t0 = time.perf_counter()
        resp = self.rollout.generate(req)
        self.rollout.sleep()
        resp.tracks["diffusion"] = self.reward.score_and_attach(req=req, track=resp.tracks["diffusion"])
        for t in resp.tracks.values():
            if t.rewards is not None:
                t.rewards = hydrate_if_handle(t.rewards)
        resp = resp.propagate_rewards(self.reward_propagation)
        mean_reward = float(resp.tracks["diffusion"].rewards.float().mean())
        results: Dict[str, Any] = {}
        for name, side in (("ar", self.ar), ("diffusion", self.diffusion)):
            track = resp.tracks[name].compute_advantages(normalize=self.normalize_adv_by_std, scope=self.adv_normalization_scope)
            track.decoded = None
            resp.tracks[name] = track
            results[name] = side["stack"].train_track(track, training_progress=float(training_progress))
        light = resp.metadata_only()
        self.wandb_logger.log_rollout_step(rollout_id, results["diffusion"], light, step_time_s=time.perf_counter() - t0,
                                           device_ms=dict(self.phase_timer.device_ms))
        return results, mean_reward

    def train(self, *, num_rollouts: int) -> None:
        self._init_wandb(num_rollouts=num_rollouts)
        try:
            for rid in range(num_rollouts):
                req = self._build_req(self.data_source.get_samples(self.batch_size), rid)
                results, mean_reward = self.train_step(req, training_progress=rid / max(1, num_rollouts - 1), rollout_id=rid)
                msg = (f"rollout {rid + 1}/{num_rollouts}  ar_loss={results['ar'].loss:.6f}  diffusion_loss={results['diffusion'].loss:.6f}  "
                       f"reward={mean_reward:.4f}")
                logger.info(msg)
                print(msg, flush=True)
        finally:
            self._finish_wandb()


__all__ = ["PETrainer"]
