"""``NativeARRolloutEngine`` — tensor-parallel paged-KV decoder replacing the external LLM servers.

The reference drives an SGLang server subprocess over HTTP (``unirl/rollout/engine/sglang_llm/engine.py:373-581``)
and pushes weights through CUDA-IPC / NCCL endpoints (``:1146-1302``).  Here the engine is a role in
the same process as the trainer shard:

* weights live in this engine's own (TP-sharded) parameter buffers, or — colocated with ``tp_size == 1``
  — alias the trainer's bf16 replica, making weight sync the identity;
* ``generate`` (``DP_SCATTER``: TP peers receive the same shard and run in lock-step; the counter-based
  sampler makes them draw identical tokens) → :class:`ARGenerator`;
* ``sleep`` / ``wake_up`` release / re-create KV cache and CUDA graphs (tags ``kv_cache`` / ``cuda_graph`` /
  ``weights`` as in the reference's memory-occupation endpoints ``:1308-1411``);
* the weight-receive surface writes full tensors through the TP slicer, or receives NCCL broadcasts.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional, Sequence

import torch

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.models.qwen3.bundle import resolve_model_config
from unirl_b200.models.qwen3.chat_template import Qwen3ChatTemplateStage, pad_right
from unirl_b200.models.qwen3.modeling import Qwen3Transformer, TPContext, shard_param, tp_slice_spec
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.models.types.contracts import unpad_prompts
from unirl_b200.models.qwen3.ar import pack_text_segment
from unirl_b200.rollout.engine.base import BaseRolloutEngine
from unirl_b200.rollout.engine.native_ar.config import NativeAREngineConfig
from unirl_b200.rollout.engine.native_ar.generator import ARGenerator
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack
from unirl_b200.types.sampling import get_ar_params
from unirl_b200.utils.dtypes import parse_torch_dtype

logger = logging.getLogger(__name__)


class NativeARRolloutEngine(BaseRolloutEngine):
    _component_name = "native_ar"

    def __init__(self, *, config: Any = None, bundle: Any = None, **overrides: Any) -> None:
        super().__init__()
        if config is None:
            config = NativeAREngineConfig(**overrides)
        elif isinstance(config, dict):
            config = NativeAREngineConfig(**{**config, **overrides})
        self.config: NativeAREngineConfig = config
        self._trainer_bundle = bundle
        self.model: Optional[Qwen3Transformer] = None
        self.generator: Optional[ARGenerator] = None
        self.tokenizer: Any = None
        self.tp_comm = None
        self.weight_version = 0
        self._shares_trainer = False
        self._sync_groups: Dict[str, Any] = {}
        self._asleep = False
        self._lora_base: Dict[str, torch.Tensor] = {}  # pristine copies of the weights that currently carry a folded-in adapter

    # ---- construction ----------------------------------------------------------------------------------
    def setup(self, *a: Any, **k: Any) -> None:
        super().setup(*a, **k)
        cfg, ri = self.config, self.rank_info
        tp = max(int(cfg.tp_size), int(ri.tp_size))
        if ri.tp_size != tp and ri.world_size > 1:
            raise ValueError(f"engine config tp_size={cfg.tp_size} but the handle was created with tp={ri.tp_size}; "
                             f"pass parallel={{'tp': {cfg.tp_size}}} to remote()")
        dev = torch.device(self.device or "cpu")
        if tp > 1:
            groups = [list(range(g * tp, (g + 1) * tp)) for g in range(ri.world_size // tp)]
            self.tp_comm = self.comm.split(groups)
            ar = self._make_all_reduce()
            tpc = TPContext(ri.tp_rank, tp, ar, fused=ar if hasattr(ar, "proj_reduce_norm") else None)
        else:
            tpc = TPContext()
        b = self._trainer_bundle
        if b is not None and tp == 1 and cfg.share_trainer_weights and getattr(b, "transformer", None) is not None:
            self.model, self._shares_trainer = b.transformer, True
            self.tokenizer = b.tokenizer
        else:
            mcfg = resolve_model_config(cfg.pretrained_model_ckpt_path, cfg.model_overrides) if b is None else b.transformer.cfg
            model_cls = type(b.transformer) if b is not None and hasattr(b.transformer, "visual") else Qwen3Transformer  # a vision-language policy keeps its vision tower
            self.model = model_cls(mcfg, dtype=parse_torch_dtype(cfg.model_precision), device=dev, tp=tpc)
            self._init_weights(b)
            self.model.eval().requires_grad_(False)
            self.tokenizer = b.tokenizer if b is not None else load_tokenizer(cfg.tokenizer_ckpt_path, mcfg.vocab_size)
        gen_kw = dict(page_size=cfg.page_size, max_running=cfg.max_running_requests, prefill_token_budget=cfg.prefill_token_budget, kv_cache_tokens=cfg.kv_cache_tokens,
                      use_cuda_graph=cfg.use_cuda_graph, poll_interval=cfg.poll_interval, seed=cfg.seed, share_prefix=bool(getattr(cfg, "share_prefix", True)))
        self._vl_pipeline = None
        if hasattr(self.model, "visual"):
            # Vision-language policy: image preprocessing, placeholder expansion and the multimodal prefill are the model package's pipeline,
            # run here on THIS engine's model (its own, possibly tensor-parallel, weights) with this engine's generator settings.
            import types

            from unirl_b200.models.qwen_vl.pipeline import QwenVLPipeline

            view = types.SimpleNamespace(transformer=self.model, tokenizer=self.tokenizer, config=b.config, model_config=self.model.cfg)
            self._vl_pipeline = QwenVLPipeline(view, detokenize=bool(cfg.detokenize), generator_kwargs=gen_kw)
            self.generator = self._vl_pipeline.ar.generator
            return
        self.generator = ARGenerator(self.model, **gen_kw)

    def _make_all_reduce(self):
        comm = self.tp_comm
        if self.config.tp_collectives == "fused" and torch.cuda.is_available():
            try:
                from unirl_b200.parallel.fused_collectives import make_fused_all_reduce

                b = self._trainer_bundle
                mcfg = b.transformer.cfg if b is not None and getattr(b, "transformer", None) is not None else \
                    resolve_model_config(self.config.pretrained_model_ckpt_path, self.config.model_overrides)
                hidden = int(mcfg.hidden_size)
                fused = make_fused_all_reduce(comm, max_tokens=max(int(self.config.prefill_token_budget), int(self.config.max_running_requests)),
                                              hidden=hidden, device=self.device)
                if fused is not None:
                    return fused
            except Exception as e:  # noqa: BLE001
                logger.warning("fused TP all-reduce unavailable (%s); using NCCL", e)
        return lambda x: comm.all_reduce(x)

    @torch.no_grad()
    def _init_weights(self, bundle: Any) -> None:
        """Random-init runs: build the *full* tensors with the trainer's seed so shards agree across TP ranks."""
        cfg, tp = self.model.cfg, self.model.tp
        if bundle is not None:
            self._load_full({n: p for n, p in bundle.transformer.named_parameters()})
            return
        if not self.config.pretrained_model_ckpt_path.startswith("random:"):
            import glob
            import os

            from safetensors.torch import load_file

            sd: Dict[str, torch.Tensor] = {}
            for f in sorted(glob.glob(os.path.join(self.config.pretrained_model_ckpt_path, "*.safetensors"))):
                sd.update(load_file(f))
            self.model.load_hf_state_dict(sd)
            return
        full = Qwen3Transformer(cfg, dtype=self.model.embed_tokens.dtype, device="cpu" if tp.size > 1 else self.model.embed_tokens.device)
        full.init_weights(self.config.init_seed)
        self._load_full(dict(full.named_parameters()))

    @torch.no_grad()
    def _load_full(self, named_full: Dict[str, torch.Tensor]) -> int:
        own = dict(self.model.named_parameters())
        tp, n = self.model.tp, 0
        for name, full in named_full.items():
            if name not in own:
                continue
            own[name].copy_(shard_param(full, name, self.model.cfg, tp.rank, tp.size).to(own[name].device))
            n += 1
        return n

    # ---- generation ----------------------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def generate(self, req: RolloutReq) -> RolloutResp:
        if self._asleep:
            self.wake_up()
        if self._vl_pipeline is not None:
            return self._vl_pipeline.generate(req)
        cond = (req.request_conditions or {}).get("prompt")
        if not isinstance(cond, TextTokenCondition):
            texts = req.primitives.get("text")
            if not isinstance(texts, Texts):
                raise TypeError("NativeARRolloutEngine.generate: need primitives['text'] (Texts) or request_conditions['prompt']")
            stage = Qwen3ChatTemplateStage(self, system_instruction=(req.stage_config.get("chat") or {}).get("system_instruction"),
                                           enable_thinking=bool(self.config.chat_template_kwargs.get("enable_thinking", False)))
            cond = stage.embed(texts).prompt
        ar = get_ar_params(req.sampling_params)
        c = self.config
        max_new = int(ar.max_new_tokens) if ar is not None else c.max_new_tokens
        temp = float(ar.temperature) if ar is not None else c.temperature
        top_p = float(ar.top_p) if ar is not None else c.top_p
        top_k = int(ar.top_k or 0) if ar is not None else c.top_k
        stop = {int(self.model.cfg.eos_token_id)}
        if ar is not None and ar.stop_token_id is not None:
            stop.add(int(ar.stop_token_id))
        prompts = unpad_prompts(cond.input_ids, cond.attention_mask)
        out = self.generator.generate(prompts, max_new_tokens=max_new, temperature=temp, top_k=top_k, top_p=top_p, stop_token_ids=sorted(stop))
        if torch.device(self.device or "cpu").type == "cuda":
            from unirl_b200.ops.status import check_device_status

            check_device_status("end of rollout batch")  # the batch's tokens were just read on the host: no extra stall
        seg = pack_text_segment(out.tokens, out.log_probs, out.finished)
        decoded = None
        if c.detokenize:
            decoded = Texts(texts=[self.tokenizer.decode(t.tolist(), skip_special_tokens=True) for t in out.tokens])
        return RolloutResp(tracks={"ar": RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids),
                                                      conditions={"prompt": cond}, segment=seg, decoded=decoded)})

    # ---- life cycle --------------------------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sleep(self, tags: Optional[Sequence[str]] = None) -> None:
        tags = set(tags or ("kv_cache", "cuda_graph"))
        if tags & {"kv_cache", "cuda_graph"} and self.generator is not None:
            self.generator.release_cache()
        if "weights" in tags and not self._shares_trainer:
            self._host_weights = {n: p.detach().to("cpu", non_blocking=True) for n, p in self.model.named_parameters()}
            for p in self.model.parameters():
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            self._lora_base = {n: t.to("cpu", non_blocking=True) for n, t in self._lora_base.items()}
        self._asleep = True

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def wake_up(self, tags: Optional[Sequence[str]] = None) -> None:
        host = getattr(self, "_host_weights", None)
        if host:
            dev = torch.device(self.device)
            for n, p in self.model.named_parameters():
                p.data = host[n].to(dev, non_blocking=True)
            self._host_weights = None
            self._lora_base = {n: t.to(dev, non_blocking=True) for n, t in self._lora_base.items()}
        self._asleep = False

    @property
    def is_offloaded(self) -> bool:
        return self._asleep

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def health_check(self) -> bool:
        return self.model is not None and self.generator is not None

    # ---- weight receive ----------------------------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def update_weights_from_tensor(self, *, serialized_named_tensors: List[Any], target_modules: Optional[List[str]] = None,
                                   load_format: Optional[str] = None, flush_cache: bool = True, track_prefix: str = "") -> int:
        """``serialized_named_tensors``: list of ``{name: full tensor}`` dicts (same process ⇒ no serialisation), every rank slicing its
        own shard out of the full tensors.  ``load_format="per_tp_rank"``: the list has one entry per tensor-parallel rank and entry ``i``
        already holds rank ``i``'s shards (the sender resharded); each rank copies its own entry as is."""
        n = 0
        if not self._shares_trainer and load_format == "per_tp_rank":
            tp = self.model.tp
            if len(serialized_named_tensors) != tp.size:
                raise ValueError(f"per_tp_rank payload has {len(serialized_named_tensors)} entries for {tp.size} tensor-parallel ranks")
            own = dict(self.model.named_parameters())
            with torch.no_grad():
                for k, v in serialized_named_tensors[tp.rank].items():
                    k = k[len(track_prefix):] if track_prefix and k.startswith(track_prefix) else k
                    if k not in own:
                        continue
                    if tuple(v.shape) != tuple(own[k].shape):
                        raise ValueError(f"per_tp_rank payload: {k} has shape {tuple(v.shape)}, this rank's shard is {tuple(own[k].shape)}")
                    own[k].copy_(v.to(own[k].device))
                    self._lora_base.pop(k, None)
                    n += 1
        elif not self._shares_trainer:
            for bucket in serialized_named_tensors:
                named = {k[len(track_prefix):] if track_prefix and k.startswith(track_prefix) else k: v for k, v in bucket.items()}
                n += self._load_full(named)
                for k in named:  # a new base replaces the one an adapter was folded into
                    self._lora_base.pop(k, None)
        self.weight_version += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    @torch.no_grad()
    def set_lora_from_tensors(self, adapter_name: str, lora_tensors: Dict[str, torch.Tensor], *, peft_config: Optional[dict] = None) -> int:
        """Install / refresh LoRA adapters from in-memory tensors keyed ``[<prefix>]model.layers.<i>.<self_attn|mlp>.<target>.lora_{A,B}[.<adapter>].weight``.

        The engine folds the adapters into its own copy of the weights: ``W[rows] = W_base[rows] + (alpha / r) * B @ A`` in fp32, for the
        row block of the fused weight the target names, sharded like the weight under tensor parallelism.  Decode therefore runs the same
        fused kernels and captured graphs as without adapters (the storage is updated in place), at the cost of one extra copy of each
        adapted weight (kept so that every sync starts from the pristine base instead of accumulating rounding).  A target that was
        adapted before and is missing from this call gets its base back.  Returns the number of adapter pairs applied.
        Parity: the engine-side half of ``unirl/distributed/weight_sync/lora/*`` (the stock engines load adapters through their own
        LoRA managers).
        """
        import re

        lora_tensors = getattr(lora_tensors, "value", lora_tensors)  # payloads pushed through the controller travel in an opaque wrapper
        self.weight_version += 1
        if self._shares_trainer:  # the trainer's module already carries the live adapters
            return 0
        pc = peft_config or {}
        scale = float(pc.get("lora_alpha", 16)) / float(pc.get("r", 8))
        c, tp = self.model.cfg, self.model.tp
        d, nq, nkv, inter = c.head_dim, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size
        where = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", nq * d), "v_proj": ("qkv_proj", (nq + nkv) * d), "o_proj": ("o_proj", 0),
                 "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", inter), "down_proj": ("down_proj", 0)}
        pat = re.compile(r"(?:^|\.)layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)\.lora_([AB])(?:\.[^.]+)?\.weight$")
        pairs: Dict[Any, Dict[str, torch.Tensor]] = {}
        for k, v in lora_tensors.items():
            m = pat.search(k)
            if m is None or m.group(2) not in where:
                continue
            pairs.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3)] = v
        by_param: Dict[str, List[Any]] = {}
        for (li, target), ab in pairs.items():
            if "A" not in ab or "B" not in ab:
                raise ValueError(f"LoRA payload has only one of lora_A / lora_B for layer {li} {target}")
            pname, off = where[target]
            by_param.setdefault(f"layers.{li}.{pname}", []).append((off, ab["A"], ab["B"]))
        own = dict(self.model.named_parameters())
        n = 0
        for name in [k for k in self._lora_base if k not in by_param]:  # adapters withdrawn: back to the base
            own[name].copy_(self._lora_base.pop(name))
        for name, parts in by_param.items():
            p = own[name]
            base = self._lora_base.get(name)
            if base is None:
                base = self._lora_base[name] = p.detach().clone()
            kind, _ = tp_slice_spec(name, c)
            rows = p.shape[0] * (tp.size if kind == "rows" else 1)
            cols = p.shape[1] * (tp.size if kind == "cols" else 1)
            delta = torch.zeros(rows, cols, dtype=torch.float32, device=p.device)
            for off, a, b in parts:
                a, b = a.to(p.device, torch.float32), b.to(p.device, torch.float32)
                if a.shape[1] != cols or off + b.shape[0] > rows or a.shape[0] != b.shape[1]:
                    raise ValueError(f"LoRA shapes A{tuple(a.shape)} B{tuple(b.shape)} do not fit {name} [{rows}, {cols}] at row {off}")
                delta[off : off + b.shape[0]].addmm_(b, a, alpha=scale)
                n += 1
            p.copy_((base.float() + shard_param(delta, name, c, tp.rank, tp.size)).to(p.dtype))
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def init_weights_update_group(self, *, src_global_rank: int, member_global_ranks: List[int], group_name: str = "weight_sync", **_kw: Any) -> None:
        """Join the trainer→engine broadcast group (built from pool-global ranks; the trainer rank joins from its side)."""
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
        dev = self.model.embed_tokens.device
        got: Dict[str, torch.Tensor] = {}
        for name, dt, shape in zip(names, dtypes, shapes):
            buf = torch.empty(shape, dtype=parse_torch_dtype(dt), device=dev)
            comm.broadcast(buf, src=self._sync_src)
            got[name] = buf
        n = self._load_full(got)
        self.weight_version += 1
        return n

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def destroy_weights_update_group(self, *, group_name: str = "weight_sync", track_prefix: str = "") -> None:
        self._sync_groups.pop(group_name, None)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def compute_local_param_checksums(self) -> Dict[str, str]:
        from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor

        return {n: fingerprint_tensor(p) for n, p in self.model.named_parameters()}

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def get_weight_version(self) -> int:
        return self.weight_version

    def shutdown(self) -> None:
        if self.generator is not None:
            self.generator.release_cache()


__all__ = ["NativeARRolloutEngine"]
