"""``NativeDiffusionRolloutEngine`` — in-process diffusion sampler with its own weights (or the trainer's, when colocated).

Takes the place of the external diffusion servers the reference drives (SGLang multimodal-gen, vLLM-Omni) and keeps
their contract: the request is authoritative for the σ schedule, the initial-noise recipe, the SDE step set and the
per-sample seeds; the engine echoes σ back and the echo is verified; trajectories are trimmed to the SDE steps; text
conditions travel back to the trainer; weights arrive in memory (full tensors, broadcast group, or LoRA tensors) and are
fingerprinted after loading; memory can be released per region (``transformer | text_encoder | vae``) while training runs.

On CUDA the denoising loop replays ONE captured graph per ``(batch, latent shape, text length)``: the transformer
forward of a step has static shapes, so after an eager first step the remaining steps cost one graph launch each.
Parity: ``unirl/rollout/engine/sglang/engine.py:115-713``, ``unirl/rollout/engine/vllm_omni/engine.py:257-1176`` and the
patch modules they install (sampling IO, set_timesteps, denoising determinism, trajectory capture, weight updaters).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from unirl_b200.config.instantiate import get_class
from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.rollout.engine.base import BaseRolloutEngine, chunked_engine_generate_req
from unirl_b200.rollout.engine.sigma_verify import verify_sigmas
from unirl_b200.sde.runtime import ensure_req_sigmas
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp
from unirl_b200.utils.dtypes import parse_torch_dtype

logger = logging.getLogger(__name__)

REGIONS = ("transformer", "text_encoder", "vae")


@dataclass
class NativeDiffusionEngineConfig:
    pipeline_cls: str = "unirl_b200.models.dit.pipeline.DiTPipeline"
    pipeline_config_cls: str = "unirl_b200.models.dit.config.DiTPipelineConfig"
    pretrained_model_ckpt_path: str = "random:tiny-sd3"
    model_precision: str = "bf16"
    autocast_precision: str = "bf16"
    device: Any = None
    share_trainer_weights: bool = True
    forward_batch_size: Optional[int] = None
    use_cuda_graph: bool = True
    verify_sigmas: bool = True
    init_seed: int = 0
    tp_size: int = 1  # tensor-parallel ranks per sampler replica (heads and MLP width of every block split; needs weights of the engine's own)
    pipeline_overrides: Dict[str, Any] = field(default_factory=dict)


class GraphedVelocity:
    """Replays the transformer evaluation of a stage (both guidance branches) from a CUDA graph once shapes are known to be static."""

    def __init__(self, stage: Any):
        self.stage = stage
        self._orig = stage._branches
        self._key: Any = None
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._x = self._sigma = self._out = None
        self._cond = self._p = None
        self._calls = 0

    def install(self) -> None:
        self.stage._branches = self.__call__

    def remove(self) -> None:
        self.stage._branches = self._orig
        self.reset()

    def reset(self) -> None:
        self._graph = None
        self._key = self._x = self._sigma = self._out = self._cond = self._p = None
        self._calls = 0

    def __call__(self, x: torch.Tensor, sigma: torch.Tensor, cond: Any, p: Any):
        if not x.is_cuda or torch.is_grad_enabled():
            return self._orig(x, sigma, cond, p)
        key = (tuple(x.shape), x.dtype, id(cond), float(p.guidance_scale))
        if key != self._key:
            self.reset()
            self._key, self._cond, self._p = key, cond, p
        self._calls += 1
        if self._calls == 1:  # eager: one-time kernel attribute and library workspace set-up happens outside capture
            return self._orig(x, sigma, cond, p)
        if self._graph is None:
            self._x, self._sigma = x.clone(), sigma.reshape(1).clone().float()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self._out = self._orig(self._x, self._sigma, self._cond, self._p)
            self._graph = g
        self._x.copy_(x)
        self._sigma.copy_(sigma.reshape(1))
        self._graph.replay()
        return tuple(None if o is None else o.clone() for o in self._out)


class NativeDiffusionRolloutEngine(BaseRolloutEngine):
    _component_name = "native_diffusion"

    def __init__(self, *, config: Any = None, pipeline: Any = None) -> None:
        super().__init__()
        self.config = config if isinstance(config, NativeDiffusionEngineConfig) else NativeDiffusionEngineConfig(**(dict(config) if config else {}))
        self._trainer_pipeline = pipeline
        self.pipeline: Any = None
        self.weight_version = 0
        self._shares_trainer = False
        self._sync_groups: Dict[str, Any] = {}
        self._host_regions: Dict[str, Dict[str, torch.Tensor]] = {}
        self._pinned: Dict[str, Dict[str, torch.Tensor]] = {}  # pinned host copies, allocated once per region and kept across sleep / wake cycles
        self._stale = set(REGIONS)  # regions whose pinned copy is older than the device weights (frozen towers are copied out once)
        self._graphed: Optional[GraphedVelocity] = None

    def setup(self, *a: Any, **k: Any) -> None:
        super().setup(*a, **k)
        c = self.config
        if self._trainer_pipeline is not None and c.share_trainer_weights:
            self.pipeline, self._shares_trainer = self._trainer_pipeline, True
        else:
            cfg_cls, pipe_cls = get_class(c.pipeline_config_cls), get_class(c.pipeline_cls)
            pcfg = cfg_cls(pretrained_model_ckpt_path=c.pretrained_model_ckpt_path, model_precision=c.model_precision, autocast_precision=c.autocast_precision,
                           device=c.device or self.device, init_seed=c.init_seed, **c.pipeline_overrides)
            self.pipeline = pipe_cls.from_config(pcfg)
            if self._trainer_pipeline is not None:  # start from the trainer's weights
                # base weights only: adapters arrive through set_lora_from_tensors
                self._load_named({n: p.detach() for n, p in self._trainer_pipeline.bundle.transformer.named_parameters() if ".lora." not in n})
            self.pipeline.bundle.transformer.eval().requires_grad_(False)
        ri = self.rank_info
        tp = max(int(c.tp_size), int(getattr(ri, "tp_size", 1) or 1))
        if tp > 1:
            if self._shares_trainer:
                raise ValueError("a tensor-parallel sampler needs weights of its own: set share_trainer_weights=false")
            if int(getattr(ri, "tp_size", 1) or 1) != tp:
                raise ValueError(f"engine config tp_size={c.tp_size} but the handle was created with tp={ri.tp_size}; pass rollout_parallel={{tp: {c.tp_size}}}")
            from unirl_b200.models.qwen3.modeling import TPContext

            self.tp_comm = self.comm.split([list(range(g * tp, (g + 1) * tp)) for g in range(ri.world_size // tp)])
            self.pipeline.bundle.transformer.apply_tensor_parallel(TPContext(ri.tp_rank, tp, lambda t: self.tp_comm.all_reduce(t)))
        self.schedule_policy = self.pipeline.build_schedule_policy()
        if c.use_cuda_graph and torch.device(self.device or "cpu").type == "cuda":
            self._graphed = GraphedVelocity(self.pipeline.diffusion)

    # ---- generate -------------------------------------------------------------------------------------------
    def _regions(self) -> Dict[str, Sequence[torch.nn.Module]]:
        b = self.pipeline.bundle
        return {"transformer": [b.transformer], "text_encoder": list(getattr(b, "text_encoders", ()) or ()), "vae": [b.vae] if getattr(b, "vae", None) is not None else []}

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def generate(self, req: RolloutReq) -> RolloutResp:
        if self._host_regions:
            self.wake_up()
        ensure_req_sigmas(req, self.schedule_policy)
        model = self.pipeline.bundle.transformer
        mode = model.training
        model.eval()
        if self._graphed is not None:
            self._graphed.install()
        try:
            with torch.no_grad():
                resp = chunked_engine_generate_req(req, self.pipeline.generate, self.config.forward_batch_size)
        finally:
            if self._graphed is not None:
                self._graphed.remove()
            model.train(mode)
        if self.config.verify_sigmas:
            for name, t in resp.tracks.items():
                if t.segment is not None and getattr(t.segment, "sigmas", None) is not None:
                    verify_sigmas(t.segment.sigmas, req.sigmas, who=f"native diffusion engine, track {name!r}")
        if torch.cuda.is_available() and any(p.is_cuda for p in model.parameters()):
            from unirl_b200.ops.status import check_device_status

            check_device_status("end of diffusion rollout batch")
        return resp

    # ---- life cycle -------------------------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sleep(self, tags: Optional[Sequence[str]] = None) -> None:
        """Release device memory of the named regions (default: the frozen aux modules; the transformer only when it is
        the engine's own copy).  Weights are stashed in pinned host memory that is allocated once and reused (pinning gigabytes takes
        seconds); a region whose weights did not change since its last stash (the text towers, the codec) is released without a copy."""
        default = ("text_encoder", "vae") if self._shares_trainer else REGIONS
        for tag in (tags or default):
            if tag not in REGIONS:
                raise ValueError(f"unknown memory region {tag!r}; regions are {REGIONS}")
            if tag in self._host_regions or (tag == "transformer" and self._shares_trainer):
                continue
            stash = self._pinned.setdefault(tag, {})
            fresh = tag not in self._stale
            found = False
            for i, mod in enumerate(self._regions()[tag]):
                for n, p in mod.named_parameters():
                    if p.device.type != "cuda":
                        continue
                    key = f"{i}.{n}"
                    host = stash.get(key)
                    if host is None or host.shape != p.shape or host.dtype != p.dtype:
                        host = stash[key] = torch.empty(p.shape, dtype=p.dtype, pin_memory=True)
                        host.copy_(p.data, non_blocking=True)
                    elif not fresh:
                        host.copy_(p.data, non_blocking=True)
                    found = True
                    p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            if found:
                self._host_regions[tag] = stash
                self._stale.discard(tag)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.empty_cache()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def wake_up(self, tags: Optional[Sequence[str]] = None) -> None:
        for tag in list(tags or self._host_regions):
            stash = self._host_regions.pop(tag, None)
            if not stash:
                continue
            for i, mod in enumerate(self._regions()[tag]):
                for n, p in mod.named_parameters():
                    key = f"{i}.{n}"
                    if key in stash:
                        p.data = stash[key].to(self.device, non_blocking=True)

    @property
    def is_offloaded(self) -> bool:
        return bool(self._host_regions)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def health_check(self) -> bool:
        return self.pipeline is not None

    # ---- weight receive ---------------------------------------------------------------------------------------
    def _load_named(self, named: Dict[str, torch.Tensor], prefix: str = "transformer.") -> int:
        self._stale.add("transformer")
        model = self.pipeline.bundle.transformer
        params = dict(model.named_parameters())
        n = 0
        with torch.no_grad():
            for k, v in named.items():
                k = k[len(prefix):] if k.startswith(prefix) else k
                if k not in params:
                    raise KeyError(f"weight {k!r} does not exist in the engine's transformer")
                if getattr(model, "tp", None) is not None:
                    v = model.tp_slice(k, v)  # full tensors arrive; a tensor-parallel rank keeps its heads / its part of the MLP width
                params[k].data.copy_(v.to(params[k].device, params[k].dtype))
                n += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def update_weights_from_tensor(self, *, serialized_named_tensors: List[Any], target_modules: Optional[List[str]] = None, load_format: Optional[str] = None,
                                   flush_cache: bool = True, track_prefix: str = "") -> int:
        n = 0
        if not self._shares_trainer:
            for bucket in serialized_named_tensors:
                n += self._load_named({(k[len(track_prefix):] if track_prefix and k.startswith(track_prefix) else k): v for k, v in bucket.items()})
        self.weight_version += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def init_weights_update_group(self, *, src_global_rank: int, member_global_ranks: List[int], group_name: str = "weight_sync", **_kw: Any) -> None:
        import torch.distributed as dist

        from unirl_b200.distributed.group.comm import Comm

        ranks = sorted(set([src_global_rank, *member_global_ranks]))
        g = dist.new_group(ranks=ranks, use_local_synchronization=True) if dist.is_initialized() and len(ranks) > 1 else None
        self._sync_groups[group_name] = Comm(g, ranks, self.comm.global_ranks[self.comm.rank] if self.comm.active else ranks[-1])
        self._sync_src = ranks.index(src_global_rank)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def update_weights_from_distributed(self, *, names: List[str], dtypes: List[str], shapes: List[List[int]], group_name: str = "weight_sync",
                                        target_modules: Optional[List[str]] = None, flush_cache: bool = True, track_prefix: str = "") -> int:
        comm = self._sync_groups[group_name]
        dev = next(self.pipeline.bundle.transformer.parameters()).device
        got: Dict[str, torch.Tensor] = {}
        for name, dt, shape in zip(names, dtypes, shapes):
            buf = torch.empty(shape, dtype=parse_torch_dtype(dt), device=dev)
            comm.broadcast(buf, src=self._sync_src)
            got[name] = buf
        n = self._load_named(got)
        self.weight_version += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def destroy_weights_update_group(self, *, group_name: str = "weight_sync", track_prefix: str = "") -> None:
        self._sync_groups.pop(group_name, None)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def set_lora_from_tensors(self, adapter_name: str, lora_tensors: Dict[str, torch.Tensor], *, peft_config: Optional[dict] = None) -> int:
        """Install / refresh LoRA adapters from in-memory tensors keyed ``<module path>.<target>.lora_{A,B}.<adapter>.weight``."""
        lora_tensors = getattr(lora_tensors, "value", lora_tensors)  # payloads pushed through the controller travel in an opaque wrapper
        from unirl_b200.train import inject

        self._stale.add("transformer")

        model = self.pipeline.bundle.transformer
        cfg = peft_config or {}
        if not any(hasattr(m, "lora") for m in model.modules()):
            inject.inject_lora(model, rank=int(cfg.get("r", 8)), alpha=float(cfg.get("lora_alpha", 16)), target_modules=tuple(cfg.get("target_modules", ())),
                               adapter_name=adapter_name, trainable=False, freeze_base=True)
        own = inject.lora_named_tensors(model, adapter_name, prefix="")
        n = 0
        with torch.no_grad():
            for k, v in lora_tensors.items():
                k = k[len("base_model.model."):] if k.startswith("base_model.model.") else k
                if k in own:
                    if getattr(model, "tp", None) is not None:
                        v = model.tp_slice(k, v)
                    own[k].data.copy_(v.to(own[k].device, own[k].dtype))
                    n += 1
        self.weight_version += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def compute_local_param_checksums(self) -> Dict[str, str]:
        from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor

        return {n: fingerprint_tensor(p) for n, p in self.pipeline.bundle.transformer.named_parameters()}

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def get_weight_version(self) -> int:
        return self.weight_version


__all__ = ["NativeDiffusionRolloutEngine", "NativeDiffusionEngineConfig", "GraphedVelocity"]
