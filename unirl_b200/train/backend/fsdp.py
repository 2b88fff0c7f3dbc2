"""``FSDPBackend`` — the sharded training backend (name kept for recipe compatibility).

Under the name lives the flat-shard runtime (``parallel/flat_shard.py``), not PyTorch FSDP2:
bf16 replica + fp32 sharded master/Adam state, per-group gradient reduce-scatter overlapped with
backward, fused AdamW, parameter publish.  The public surface follows
``unirl/train/backend/fsdp.py``: construction order (adapter injection → sharding → materialise →
EMA → optimizer → schedule) ``:66-189``; ``zero_grad`` / ``set_grad_sync`` / ``optimizer_step`` (clip, skip
on a non-finite norm, step, schedule, EMA) ``:195-267``; ``save`` / ``load`` with the same ``checkpoint.pt``
dict ``:301-388``; ``offload`` / ``onload`` ``:394-419``; checksum and smoke helpers ``:432-482``.
"""

from __future__ import annotations

import hashlib
import logging
import math
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.distributed.group.remote import Remote
from unirl_b200.parallel.flat_shard import FlatShardedModel
from unirl_b200.train.configs import EmaFullConfig, EmaLoraConfig, FSDPConfig, LoraConfig, LrSchedulerConfig, OptimizerConfig
from unirl_b200.train.ema import ShardEMA
from unirl_b200.train.factories import build_lr_scheduler
from unirl_b200.utils.dtypes import parse_torch_dtype

logger = logging.getLogger(__name__)


def _as_cfg(cls: type, value: Any) -> Any:
    if value is None or isinstance(value, cls):
        return value
    return cls(**{k: v for k, v in dict(value).items() if not k.startswith("_")})


class FSDPBackend(Remote):
    def __init__(self, *, bundle: Any, block_class_names: Sequence[str] = (), fsdp_cfg: Any = None, optimizer_cfg: Any = None,
                 scheduler_cfg: Any = None, device: Optional[Any] = None, rank: int = 0, trainable_attr: str = "transformer",
                 lora_cfg: Any = None, ema_lora_cfg: Any = None, ema_cfg: Any = None, with_aux: Sequence[str] = ()) -> None:
        super().__init__()
        self.fsdp_cfg: FSDPConfig = _as_cfg(FSDPConfig, fsdp_cfg) or FSDPConfig()
        self.optimizer_cfg: OptimizerConfig = _as_cfg(OptimizerConfig, optimizer_cfg) or OptimizerConfig()
        self.scheduler_cfg: LrSchedulerConfig = _as_cfg(LrSchedulerConfig, scheduler_cfg) or LrSchedulerConfig()
        self.lora_cfg, self.ema_lora_cfg, self.ema_cfg = _as_cfg(LoraConfig, lora_cfg), _as_cfg(EmaLoraConfig, ema_lora_cfg), _as_cfg(EmaFullConfig, ema_cfg)
        if self.lora_cfg is not None and self.ema_lora_cfg is not None:
            raise ValueError("FSDPBackend: lora_cfg and ema_lora_cfg are mutually exclusive")
        self._bundle, self._trainable_attr = bundle, trainable_attr
        self._block_class_names, self._with_aux = tuple(block_class_names), tuple(with_aux)
        self._forced_device = device
        self.model: nn.Module = getattr(bundle, trainable_attr)
        self.sharded: Optional[FlatShardedModel] = None
        self.ema: Optional[Any] = None
        self.scheduler = build_lr_scheduler(self.scheduler_cfg, self.optimizer_cfg.learning_rate)
        self._optimizer_step_count = 0
        self._eval_ema_active = False
        self._defer_grad_sync = True  # grads always accumulate locally; one reduce-scatter per optimizer step
        active = self.lora_cfg or self.ema_lora_cfg
        self._lora_meta = ({"rank": int(active.rank), "alpha": int(active.alpha), "target_modules": list(active.target_modules)}
                           if active is not None else None)
        self._built = False

    # ---- construction (needs the role's comm, so it completes in setup) --------------------------------
    def setup(self, *a: Any, **k: Any) -> None:
        super().setup(*a, **k)
        self._build()

    def _build(self) -> None:
        if self._built:
            return
        from unirl_b200.train import inject

        dev = torch.device(self._forced_device or self.device or ("cuda" if torch.cuda.is_available() else "cpu"))
        shadow = None
        if self.ema_lora_cfg is not None:
            c = self.ema_lora_cfg
            shadow = inject.inject_nft(self.model, rank=c.rank, alpha=c.alpha, target_modules=tuple(c.target_modules),
                                       default=c.default_adapter, shadow=c.shadow_adapter, dropout=c.dropout)
        elif self.lora_cfg is not None:
            c = self.lora_cfg
            inject.inject_lora(self.model, rank=c.rank, alpha=c.alpha, target_modules=tuple(c.target_modules), dropout=c.dropout)
        mat = getattr(self._bundle, "materialize", None)
        if callable(mat):
            mat(device=dev, with_aux=self._with_aux)
        self.model.to(dev)
        if self.fsdp_cfg.activation_checkpointing and hasattr(self.model, "gradient_checkpointing"):
            self.model.gradient_checkpointing = True
            if hasattr(self.model, "checkpoint_layers"):
                self.model.checkpoint_layers = self.fsdp_cfg.checkpoint_layers
        low = parse_torch_dtype(self.fsdp_cfg.param_dtype) if self.fsdp_cfg.mixed_precision else next(self.model.parameters()).dtype
        if dev.type == "cpu" and not self.fsdp_cfg.mixed_precision:
            low = next(self.model.parameters()).dtype
        blocks = self._block_class_names or tuple(getattr(self.model, "_no_split_modules", ()) or ())
        sp = int(getattr(self.fsdp_cfg, "sp_size", 1) or 1)
        if sp > 1:
            from unirl_b200.parallel.ulysses import UlyssesContext

            if self.comm.size % sp:
                raise ValueError(f"sp_size={sp} does not divide the trainer's {self.comm.size} ranks")
            if self.rank_info.sp_size != sp:
                raise ValueError(f"fsdp_cfg.sp_size={sp} but the role was placed with sp={self.rank_info.sp_size}; pass train_parallel={{sp: {sp}}}")
            groups = [list(range(g * sp, (g + 1) * sp)) for g in range(self.comm.size // sp)]
            ctx = UlyssesContext(self.comm.split(groups))
            for m in self.model.modules():
                if hasattr(m, "sp") and hasattr(m, "patchify"):
                    m.sp = ctx
        cp = int(getattr(self.fsdp_cfg, "cp_size", 1) or 1)
        if cp > 1:
            # Context parallelism of the autoregressive replay: the ranks of a group see the SAME sequences (placed like sequence-parallel
            # peers: train_parallel={sp: cp}) and each runs its chunk of every sequence; partial gradients add up like under sp.
            from unirl_b200.parallel.context_parallel import ContextParallel

            if sp > 1:
                raise ValueError("sp_size and cp_size are not combined")
            if self.comm.size % cp:
                raise ValueError(f"cp_size={cp} does not divide the trainer's {self.comm.size} ranks")
            if self.rank_info.sp_size != cp:
                raise ValueError(f"fsdp_cfg.cp_size={cp} but the role was placed with sp={self.rank_info.sp_size}; pass train_parallel={{sp: {cp}}}")
            targets = [m for m in self.model.modules() if hasattr(m, "cp") and hasattr(m, "embed_tokens")]
            if not targets:
                raise ValueError("cp_size > 1 needs a model with a context-parallel replay (the autoregressive decoders)")
            ctx = ContextParallel(self.comm.split([list(range(g * cp, (g + 1) * cp)) for g in range(self.comm.size // cp)]))
            for m in targets:
                m.cp = ctx
            sp = cp  # gradient bookkeeping below: partial gradients of `cp` peers add up
        shard_group, replicate_group = self.comm, None
        hs = int(self.fsdp_cfg.hsdp_shard_size)
        if self.fsdp_cfg.fsdp_mode == "hybrid" and self.comm.size > hs and self.comm.size % hs == 0:
            n_rep = self.comm.size // hs
            shard_group = self.comm.split([list(range(r * hs, (r + 1) * hs)) for r in range(n_rep)])
            replicate_group = self.comm.split([[r * hs + i for r in range(n_rep)] for i in range(hs)])
        self._shard_group = shard_group
        zero3 = bool(self.fsdp_cfg.reshard_after_forward) and shard_group.active
        self.sharded = FlatShardedModel(self.model, shard_group, block_class_names=blocks, root_wrap=self.fsdp_cfg.root_wrap,
                                        reshard_after_forward=zero3, replicate_comm=replicate_group, low_dtype=low, trainable_only=False, grad_replicas=sp,
                                        shard_comm=self._make_shard_comm())
        if shadow is not None:
            shadow.bind(self.sharded)
            c = self.ema_lora_cfg
            shadow.configure(decay=c.ema_decay, decay_type=c.ema_decay_type, timing=c.timing, flat_steps=c.ema_flat_steps,
                             uprate=c.ema_uprate, uphold=c.ema_uphold)
            self.ema = shadow
        elif self.ema_cfg is not None:
            self.ema = ShardEMA(self.sharded, self.ema_cfg.target_decay, self.ema_cfg.timing)
        self._built = True

    def _make_shard_comm(self) -> Any:
        fused_ok = not self.fsdp_cfg.reshard_after_forward and self.fsdp_cfg.fsdp_mode != "hybrid"  # peer arenas are never released and span one group
        if fused_ok and self.fsdp_cfg.collectives == "fused" and self.comm.active and torch.cuda.is_available():
            try:
                from unirl_b200.parallel.fused_collectives import FusedShardComm

                return FusedShardComm(self.comm)
            except Exception as e:  # noqa: BLE001 - the NCCL path is a complete implementation
                logger.warning("fused collectives unavailable (%s); using NCCL", e)
        return None

    # ---- step protocol ---------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.sharded.release_all()  # ZeRO-3: replicas live only around their block while a train step runs (no-op otherwise)
        self.sharded.zero_grad()

    def set_grad_sync(self, enable: bool) -> None:
        self.sharded.set_grad_sync(enable)

    @property
    def grad_sync_deferred(self) -> bool:
        return self._defer_grad_sync

    @property
    def current_lr(self) -> float:
        return self.scheduler.lr

    def any_rank(self, flag: bool) -> bool:
        """``flag`` OR-ed over the trainer's ranks: whether to take an optimizer step is one decision for the whole group (a rank
        whose micro-batches were all empty still joins the reductions with zero gradients)."""
        if not self.comm.active:
            return bool(flag)
        t = torch.tensor([1.0 if flag else 0.0], device=self.sharded.device)
        self.comm.all_reduce(t, op="max")
        return bool(t.item() > 0)

    def optimizer_step(self, *, max_grad_norm: float) -> float:
        """Clip by global norm, skip on a non-finite norm (identical verdict on every rank), step, schedule, EMA."""
        sh, oc = self.sharded, self.optimizer_cfg
        sh.finish_grad_sync()
        norm_t = sh.grad_norm()
        grad_norm = float(norm_t)  # the one host sync of the step: also the skip verdict
        sh.shard_comm.check()  # a peer wait that ran out of time raises here instead of training on a partial reduction
        if sh.device.type == "cuda":
            from unirl_b200.ops.status import check_device_status

            check_device_status("optimizer step")  # GEMM / attention status word and every live peer arena
        if not math.isfinite(grad_norm):
            logger.warning("non-finite grad norm (%s) at optimizer step %d; skipping the update", grad_norm, self._optimizer_step_count)
            sh.zero_grad()
            return grad_norm
        coef = torch.clamp(max_grad_norm / (norm_t + 1e-6), max=1.0).float().reshape(1)
        ema_decay = None
        if isinstance(self.ema, ShardEMA) and self.ema.timing == "optimizer_step":
            ema_decay = self.ema.decay(self._optimizer_step_count)
        sh.optimizer_step(lr=self.scheduler.lr, betas=(oc.adam_beta1, oc.adam_beta2), eps=oc.adam_epsilon, weight_decay=oc.weight_decay,
                          step=self._optimizer_step_count + 1, clip_coef=coef, ema_decay=ema_decay)
        self.scheduler.step()
        if self.ema is not None and not isinstance(self.ema, ShardEMA):
            self.ema.step(self._optimizer_step_count)
        self._optimizer_step_count += 1
        return grad_norm

    def on_rollout_end(self) -> None:
        if self.ema is not None:
            self.ema.on_rollout_end(self._optimizer_step_count)
        self.sharded.release_grad_buffers()
        self.sharded.gather_all()  # ZeRO-3: rollout, weight sync and checkpointing see whole parameters

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def apply_eval_ema(self) -> None:
        if self.ema is None or self._eval_ema_active:
            return
        self.ema.apply_shadow()
        self._eval_ema_active = True

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def restore_from_eval(self) -> None:
        if self.ema is None or not self._eval_ema_active:
            return
        self.ema.restore_shadow()
        self._eval_ema_active = False

    # ---- state dicts -------------------------------------------------------------------------------------
    def policy_state_dict(self) -> Dict[str, torch.Tensor]:
        from unirl_b200.train.fsdp_utils import full_state_dict

        return full_state_dict(self.model)

    def raw_named_params(self):
        return self.sharded.named_full_params()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def save(self, path: str, step: Optional[int] = None, mode: str = "full") -> None:
        if mode not in ("full", "adapter"):
            raise ValueError(f"FSDPBackend.save: unknown mode {mode!r}")
        sd = {k: v.detach().cpu().clone() for k, v in self.policy_state_dict().items()}
        if mode == "adapter":
            sd = {k: v for k, v in sd.items() if "lora_A" in k or "lora_B" in k}
            if not sd:
                raise RuntimeError("FSDPBackend.save: mode='adapter' but the model has no LoRA parameters")
        opt = self.sharded.optimizer_state_dict()  # collective
        state = {"policy_state_dict": sd, "optimizer_state_dict": {"state": opt, "param_groups": [self._param_group_dict()]},
                 "optimizer_step_count": self._optimizer_step_count, "step": step, "save_mode": mode, "lora_config": self._lora_meta,
                 "scheduler_state_dict": self.scheduler.state_dict()}
        if self.rank_info.rank != 0:
            return
        os.makedirs(path, exist_ok=True)
        tmp = os.path.join(path, "checkpoint.pt.tmp")
        torch.save(state, tmp)
        os.replace(tmp, os.path.join(path, "checkpoint.pt"))
        from unirl_b200.train.fsdp_utils import write_manifest

        write_manifest(path, sd)

    def _param_group_dict(self) -> Dict[str, Any]:
        oc = self.optimizer_cfg
        return {"lr": self.scheduler.lr, "betas": (oc.adam_beta1, oc.adam_beta2), "eps": oc.adam_epsilon, "weight_decay": oc.weight_decay}

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def load(self, path: str) -> int:
        ckpt_path = os.path.join(path, "checkpoint.pt")
        seen = self.comm.all_gather_object(os.path.exists(ckpt_path))  # agree BEFORE any collective so no rank hangs
        missing = [r for r, ok in enumerate(seen) if not ok]
        if missing:
            raise FileNotFoundError(f"FSDPBackend.load: checkpoint not visible on rank(s) {missing}: {ckpt_path}")
        ckpt = torch.load(ckpt_path, map_location="cpu", weights_only=False)
        from unirl_b200.train.fsdp_utils import load_full_state_dict

        load_full_state_dict(self.model, ckpt["policy_state_dict"], strict=ckpt.get("save_mode", "full") == "full")
        self.sharded.sync_master_from_params()
        self.sharded.load_optimizer_state_dict(ckpt["optimizer_state_dict"].get("state", {}))
        if "scheduler_state_dict" in ckpt:
            self.scheduler.load_state_dict(ckpt["scheduler_state_dict"])
        if ckpt.get("optimizer_step_count") is not None:
            self._optimizer_step_count = int(ckpt["optimizer_step_count"])
        return int(ckpt.get("step") or 0)

    # ---- colocate memory dance -----------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def offload(self) -> None:
        self.sharded.offload()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def onload(self) -> None:
        self.sharded.onload()

    # ---- verification helpers --------------------------------------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def compute_local_param_checksums(self) -> Dict[str, str]:
        from unirl_b200.distributed.weight_sync.checksum import fingerprint_tensor

        return {n: fingerprint_tensor(p) for n, p in self.sharded.named_full_params()}

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def randomize_weights_for_smoke(self, seed: int = 1234, scale: float = 0.02) -> None:
        g = torch.Generator().manual_seed(int(seed))
        with torch.no_grad():
            for _n, p in self.sharded.named_full_params():
                p.copy_((torch.randn(p.shape, generator=g) * scale).to(p))
        self.sharded.sync_master_from_params()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def memory_info(self) -> Dict[str, float]:
        out = {"train_state_gb": self.sharded.state_bytes() / 2**30}
        if torch.cuda.is_available():
            out["cuda_allocated_gb"] = torch.cuda.memory_allocated() / 2**30
            out["cuda_reserved_gb"] = torch.cuda.memory_reserved() / 2**30
        return out


__all__ = ["FSDPBackend"]
