"""Flat sharded-parameter runtime: the FSDP2 replacement, designed around 180 GB of HBM per GPU.

Layout per *group* (one decoder / DiT block, or the root group of embeddings + head):

``flat_param``  bf16  ``[P]``     every parameter of the group back to back (each padded to 8 elements, the
                                 whole padded to a multiple of ``world·ALIGN``); module parameters are *views*
``main_grad``   fp32  ``[P]``     gradient accumulator across micro-batches (allocated for the train phase only)
``master`` / ``exp_avg`` / ``exp_avg_sq``  fp32 ``[P / world]``  this rank's optimizer shard

Two residency modes:

* ``reshard_after_forward=False`` (ZeRO-2, default): the bf16 replica stays resident (8 GB for a 4 B
  model is cheap on B200), so forward/backward issue **no** parameter collectives; after the
  optimizer step every rank republishes its updated bf16 shard (one all-gather per step — or, on
  the fused path, the AdamW kernel stores its shard straight into every peer's replica).
* ``reshard_after_forward=True`` (ZeRO-3): only the local shard is resident between uses; groups
  are gathered around their forward/backward (the next block's gather is prefetched on a side stream).

Gradient path: per-parameter post-accumulate hooks fold the bf16 autograd gradient into the fp32
``main_grad`` view; when the last micro-batch finishes a group, its reduce-scatter is launched on the
communication stream (overlapping the rest of backward) — in a fixed group order that is the same on every
rank, whichever parameters received gradients there; the optimizer step then runs one fused
AdamW kernel per group over the flat shard with the clip coefficient read from a device scalar.

The collectives go through a small ``ShardComm`` strategy object so the NCCL implementation (the
measured baseline) and the fused peer-memory kernels (``parallel/fused_collectives.py``) are
interchangeable.  Reference behaviour being replaced: ``unirl/train/inject.py:189-383`` (``fully_shard``
per block, mixed precision bf16 params / fp32 reduce), ``unirl/train/fsdp_utils.py:274-319`` (clip).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.ops import optim as O

ALIGN = 128  # elements; keeps every shard boundary 256-byte aligned in bf16 (TMA / vector friendly)


def _pad(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: Tuple[int, ...]


class ShardComm:
    """NCCL/gloo baseline collectives for the sharded runtime.

    A subclass may also own the memory of the replicas and gradient buffers (``reserve`` / ``alloc_param`` /
    ``alloc_grad``) and fold the parameter publish into the optimizer kernel (``fused_optimizer``).
    """

    fused_optimizer = False
    persistent_grads = False

    def __init__(self, comm: Comm):
        self.comm = comm

    def reserve(self, param_bytes: int, grad_bytes: int, device: Any) -> None:
        """Called once with the total bytes of all replicas / gradient buffers before any group is built."""

    def alloc_param(self, numel: int, dtype: torch.dtype, device: Any) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=device)

    def alloc_grad(self, numel: int, device: Any) -> torch.Tensor:
        return torch.zeros(numel, dtype=torch.float32, device=device)

    def begin_grad_sync(self) -> None:
        """Called when the last micro-batch of a step starts (before any reduce-scatter of that step)."""

    def local_sumsq(self) -> Optional[torch.Tensor]:
        """Σ of squared reduced gradients of this rank's shards if the reduce kernels accumulated it, else None."""
        return None

    def check(self) -> None:
        """Raise if a device-side wait failed since the last check (no-op for library collectives)."""

    def reduce_scatter_grad(self, group: "FlatGroup") -> None:
        """``main_grad`` (fp32, full) → ``grad_shard`` (fp32, averaged over ranks)."""
        self.comm.reduce_scatter_into(group.grad_shard, group.main_grad, op="avg")

    def publish_params(self, group: "FlatGroup") -> None:
        """Every rank's updated bf16 shard → every rank's full replica."""
        if self.comm.active:
            self.comm.all_gather_into(group.flat_param, group.param_shard.clone())

    def gather_params(self, group: "FlatGroup", out: torch.Tensor) -> None:
        self.comm.all_gather_into(out, group.param_shard_resident)


class FlatGroup:
    def __init__(self, name: str, named_params: Sequence[Tuple[str, nn.Parameter]], rank: int, world: int, device: Any,
                 low_dtype: torch.dtype = torch.bfloat16, master_dtype: torch.dtype = torch.float32, alloc: Optional[ShardComm] = None):
        self.name, self.rank, self.world = name, rank, world
        self._alloc = alloc
        self._persist_grad: Optional[torch.Tensor] = None
        self.low_dtype, self.master_dtype = low_dtype, master_dtype
        self.slots: List[ParamSlot] = []
        off = 0
        for n, p in named_params:
            self.slots.append(ParamSlot(n, p, off, p.numel(), tuple(p.shape)))
            off += _pad(p.numel(), 8)
        self.numel = off
        self.padded = self.padded_numel(named_params, world)
        self.shard_size = self.padded // world
        dev = torch.device(device)
        self.flat_param = alloc.alloc_param(self.padded, low_dtype, dev) if alloc is not None else torch.zeros(self.padded, dtype=low_dtype, device=dev)
        for s in self.slots:
            view = self.flat_param[s.offset : s.offset + s.numel].view(s.shape)
            view.copy_(s.param.data.to(low_dtype))
            s.param.data = view
        lo, hi = rank * self.shard_size, (rank + 1) * self.shard_size
        self.param_shard = self.flat_param[lo:hi]
        self.master = self.param_shard.to(master_dtype).clone()
        self.exp_avg = torch.zeros(self.shard_size, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard_size, dtype=torch.float32, device=dev)
        self.main_grad: Optional[torch.Tensor] = None
        self.grad_shard: Optional[torch.Tensor] = None
        self.ema: Optional[torch.Tensor] = None
        self._pending = 0
        self._hooks: List[Any] = []
        self.trainable = any(s.param.requires_grad for s in self.slots)
        self.expert_local = False  # parameters owned by this expert-parallel rank: never reduced, sharded or published
        self.module: Optional[nn.Module] = None  # the block whose forward / backward brackets the gather (ZeRO-3)
        self.shard_resident: Optional[torch.Tensor] = None  # ZeRO-3: this rank's bf16 shard while the replica storage is released
        self._gathered = True
        self._fetch: Any = None  # a gather in flight: True (issued inline) or the event recorded on the prefetch stream

    # ---- ZeRO-3 residency ---------------------------------------------------------------------------
    def release_replica(self) -> None:
        """Keep only this rank's shard; the replica's storage is handed back to the allocator (views stay valid objects)."""
        self.join_fetch()
        if not self._gathered:
            return
        if self.shard_resident is None:
            self.shard_resident = self.param_shard.clone()
        else:
            self.shard_resident.copy_(self.param_shard)
        self.flat_param.untyped_storage().resize_(0)
        self._gathered = False

    def start_fetch(self, gather: Callable[[torch.Tensor, torch.Tensor], None], stream: Any = None) -> None:
        """Begin rebuilding the replica from the shards: on ``stream`` when given (prefetch, the caller's stream goes on), else inline."""
        if self._gathered or self._fetch is not None:
            return
        self.flat_param.untyped_storage().resize_(self.padded * self.flat_param.element_size())
        if stream is None:
            gather(self.flat_param, self.shard_resident)
            self._fetch = True
        else:
            stream.wait_stream(torch.cuda.current_stream())  # the storage was just handed out in the caller's stream order
            with torch.cuda.stream(stream):
                gather(self.flat_param, self.shard_resident)
            self._fetch = stream.record_event()

    def join_fetch(self) -> None:
        """Make a fetch in flight visible to the current stream."""
        if self._fetch is None:
            return
        if self._fetch is not True:
            torch.cuda.current_stream().wait_event(self._fetch)
        self._fetch = None
        self._gathered = True

    def restore_replica(self, gather: Callable[[torch.Tensor, torch.Tensor], None]) -> None:
        self.start_fetch(gather)
        self.join_fetch()

    @staticmethod
    def padded_numel(named_params: Sequence[Tuple[str, nn.Parameter]], world: int) -> int:
        return _pad(max(sum(_pad(p.numel(), 8) for _, p in named_params), 1), world * ALIGN)

    # ---- gradient buffers -----------------------------------------------------------------------
    def ensure_grad_buffers(self) -> None:
        if self.main_grad is None:
            dev = self.flat_param.device
            if self._alloc is not None and self._alloc.persistent_grads:
                if self._persist_grad is None:
                    self._persist_grad = self._alloc.alloc_grad(self.padded, dev)
                else:
                    self._persist_grad.zero_()
                self.main_grad = self._persist_grad
            else:
                self.main_grad = torch.zeros(self.padded, dtype=torch.float32, device=dev)
            self.grad_shard = torch.zeros(self.shard_size, dtype=torch.float32, device=dev) if self.world > 1 else \
                self.main_grad[: self.shard_size]

    def release_grad_buffers(self) -> None:
        self.main_grad = self.grad_shard = None

    def grad_view(self, slot: ParamSlot) -> torch.Tensor:
        return self.main_grad[slot.offset : slot.offset + slot.numel].view(slot.shape)

    def shard_range(self) -> Tuple[int, int]:
        return self.rank * self.shard_size, (self.rank + 1) * self.shard_size

    def state_bytes(self) -> int:
        n = self.flat_param.numel() * self.flat_param.element_size() + 3 * self.shard_size * 4
        return n + (self.main_grad.numel() * 4 if self.main_grad is not None else 0)


class FlatShardedModel:
    """Owns the groups of one trainable module and drives grad sync + optimizer + publish."""

    def __init__(self, module: nn.Module, comm: Optional[Comm] = None, *, block_class_names: Sequence[str] = (), root_wrap: bool = True,
                 reshard_after_forward: bool = False, low_dtype: torch.dtype = torch.bfloat16, master_dtype: torch.dtype = torch.float32,
                 shard_comm: Optional[ShardComm] = None, trainable_only: bool = False, grad_replicas: int = 1, replicate_comm: Optional[Comm] = None):
        self.module = module
        # HSDP: `comm` is the SHARD group (parameters / optimizer state are sharded inside it), `replicate_comm` links the ranks that
        # own the same shard in different replicas; gradients are reduce-scattered inside the shard group, then all-reduced across replicas.
        self.replicate_comm = replicate_comm if replicate_comm is not None and replicate_comm.active else None
        self.comm = comm or Comm.solo()
        self.rank, self.world = max(self.comm.rank, 0), self.comm.size
        self.reshard_after_forward = bool(reshard_after_forward)
        self.shard_comm = shard_comm or ShardComm(self.comm)
        # Sequence / tensor-parallel peers see the SAME samples and hold PARTIAL gradients of them: their contributions add up,
        # only the data-parallel replicas are averaged.  The reduce averages over all ranks, so gradients are rescaled by this factor.
        self.grad_replicas = max(1, int(grad_replicas))
        self.device = next(module.parameters()).device
        self.groups: List[FlatGroup] = []
        self._sync_enabled = True
        self._norm_sq: Optional[torch.Tensor] = None
        self._comm_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" and self.world > 1 else None
        self._reduce_on_ready = True  # ZeRO-2: a group is reduced as soon as its hooks have fired and its turn has come
        self._schedule: Optional[List[FlatGroup]] = None
        self._cursor = 0
        self._build_groups(block_class_names, root_wrap, low_dtype, master_dtype, trainable_only)
        self._install_hooks()
        if self.reshard_after_forward and self.world > 1:
            self._install_zero3_hooks()

    # ---- construction ----------------------------------------------------------------------------
    def _build_groups(self, block_names: Sequence[str], root_wrap: bool, low: torch.dtype, master: torch.dtype, trainable_only: bool) -> None:
        taken: set = set()
        want = set(block_names)
        layout: List[Tuple[str, List[Tuple[str, nn.Parameter]]]] = []
        for mod_name, mod in self.module.named_modules():
            if type(mod).__name__ in want:
                named = [(f"{mod_name}.{n}", p) for n, p in mod.named_parameters() if id(p) not in taken and (p.requires_grad or not trainable_only)]
                if named:
                    taken.update(id(p) for _, p in named)
                    layout.append((mod_name, named))
        rest = [(n, p) for n, p in self.module.named_parameters() if id(p) not in taken and (p.requires_grad or not trainable_only)]
        if rest:
            if not root_wrap and any(p.requires_grad for _, p in rest) and self.world > 1:
                raise ValueError("root_wrap=False leaves trainable parameters outside every sharded group: "
                                 + ", ".join(n for n, p in rest if p.requires_grad)[:200])
            layout.insert(0, ("<root>", rest))
        # parameters owned by one expert-parallel rank (not replicated) get groups of their own: no reduction, no sharding, local update
        split: List[Tuple[str, List[Tuple[str, nn.Parameter]]]] = []
        self._ep_group_names: set = set()
        for name, named in layout:
            rep = [(n, p) for n, p in named if not getattr(p, "_ep_local", False)]
            loc = [(n, p) for n, p in named if getattr(p, "_ep_local", False)]
            if rep:
                split.append((name, rep))
            if loc:
                split.append((name + "#experts", loc))
                self._ep_group_names.add(name + "#experts")
        layout = split
        sizes = [FlatGroup.padded_numel(named, 1 if name in self._ep_group_names else self.world) for name, named in layout]
        low_bytes = torch.empty((), dtype=low).element_size()
        self.shard_comm.reserve(sum(s * low_bytes + 256 for s in sizes),
                                sum(s * 4 + 256 for s, (_, named) in zip(sizes, layout) if any(p.requires_grad for _, p in named)), self.device)
        modules = dict(self.module.named_modules())
        for name, named in layout:
            if name in self._ep_group_names:
                g = FlatGroup(name, named, 0, 1, self.device, low, master, alloc=None)
                g.expert_local = True
                self.groups.append(g)
                continue
            self.groups.append(FlatGroup(name, named, self.rank, self.world, self.device, low, master, alloc=self.shard_comm))
            self.groups[-1].module = modules.get(name)
        if self.world > 1 and self.shard_comm.persistent_grads:
            for g in self.groups:  # symmetric layout: every rank allocates in the same order
                if g.trainable and not g.expert_local:
                    g._persist_grad = self.shard_comm.alloc_grad(g.padded, self.device)

    def _install_hooks(self) -> None:
        for g in self.groups:
            for s in g.slots:
                if s.param.requires_grad:
                    g._hooks.append(s.param.register_post_accumulate_grad_hook(self._make_hook(g, s)))
                    # Linear layers that find this attribute accumulate their weight gradient straight into the fp32 buffer
                    # (GEMM with beta = 1) instead of materialising a bf16 gradient that the hook then adds.
                    s.param._wgrad_accum = self._make_accum(g, s)

    @staticmethod
    def _make_accum(g: FlatGroup, s: ParamSlot) -> Callable[[], torch.Tensor]:
        def accum() -> torch.Tensor:
            g.ensure_grad_buffers()
            return g.grad_view(s)

        return accum

    # ---- ZeRO-3: replicas exist only around their block's forward and backward ------------------------------------
    def _gather_into(self, out: torch.Tensor, shard: torch.Tensor) -> None:
        self.comm.all_gather_into(out, shard)

    def _install_zero3_hooks(self) -> None:
        """Block groups release their replica after forward and after backward and gather it back before either; while block i
        computes, the gather of the block that runs next (i+1 in forward, i-1 in backward) is already in flight on a side stream.
        The root group (embeddings, final norm, head) stays resident: it is used at both ends of every pass.

        Every collective of this mode is issued from a module hook, so its position in the sequence of collectives does not depend
        on which parameters received gradients: gathers at block entry, and the reduce-scatter of every block after block i
        when block i's backward begins (the rest at ``finish_grad_sync``).  All ranks must run the same micro-batches."""
        if getattr(self.shard_comm, "persistent_grads", False):
            raise ValueError("reshard_after_forward=True needs the library collectives (replica storage is released between uses)")
        self._z3_blocks = [g for g in self.groups if g.module is not None and g.module is not self.module]
        self._z3_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._z3_in_backward = False
        self._reduce_on_ready = False
        for i, g in enumerate(self._z3_blocks):
            g._hooks.append(g.module.register_forward_pre_hook(lambda _m, _a, i=i: self._z3_forward_pre(i)))
            g._hooks.append(g.module.register_forward_hook(lambda _m, _a, _o, i=i: self._z3_forward_post(i)))
            g._hooks.append(g.module.register_full_backward_pre_hook(lambda _m, _go, i=i: self._z3_backward_pre(i)))
            g.release_replica()

    def _z3_enter(self, i: int, step: int) -> None:
        blocks = self._z3_blocks
        blocks[i].start_fetch(self._gather_into)  # not prefetched (first block of a pass): gather in the compute stream
        blocks[i].join_fetch()
        j = i + step
        if step and 0 <= j < len(blocks):
            blocks[j].start_fetch(self._gather_into, self._z3_stream)

    def _z3_forward_pre(self, i: int) -> None:
        # inside backward this is the recomputation of a checkpointed block: its backward-pre hook already fetched it and its successor
        self._z3_enter(i, 0 if self._z3_in_backward else 1)

    def _z3_forward_post(self, i: int) -> None:
        if not self._z3_in_backward:  # a recomputed block is about to run its backward: keep it
            self._z3_blocks[i].release_replica()

    def _z3_backward_pre(self, i: int) -> None:
        if not self._z3_in_backward:
            self._z3_in_backward = True
            torch.autograd.Variable._execution_engine.queue_callback(self._z3_backward_done)
        self._z3_enter(i, -1)
        if self._sync_enabled and self.world > 1:
            self._drain_schedule(force=True, before=self._z3_blocks[i])
        for g in self._z3_blocks[i + 1:]:  # blocks whose backward is complete
            g.release_replica()

    def _z3_backward_done(self) -> None:
        self._z3_in_backward = False
        for g in self._z3_blocks:
            g.release_replica()

    def gather_all(self) -> None:
        """Make every replica resident (checkpoint save, weight sync, rollout on the trainer's module)."""
        for g in self.groups:
            g.restore_replica(self._gather_into)

    def release_all(self) -> None:
        if self.reshard_after_forward and self.world > 1:
            for g in self.groups:
                if g.module is not None and g.module is not self.module:
                    g.release_replica()

    def _make_hook(self, g: FlatGroup, s: ParamSlot) -> Callable[[torch.Tensor], None]:
        def hook(p: torch.Tensor) -> None:
            if p.grad is None:
                return
            g.ensure_grad_buffers()
            if getattr(p, "_wgrad_fused", False):
                p._wgrad_fused = False  # the producing GEMM already added into the fp32 buffer; p.grad is a placeholder
            else:
                g.grad_view(s).add_(p.grad)
            p.grad = None
            if self._sync_enabled and self.world > 1:
                g._pending -= 1
                if g._pending == 0:
                    g._ready = True
                    if self._reduce_on_ready:
                        self._drain_schedule()

        return hook

    # ---- step protocol ------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        for g in self.groups:
            if g.main_grad is not None:
                g.main_grad.zero_()
            for s in g.slots:
                s.param.grad = None

    def set_grad_sync(self, enable: bool) -> None:
        """``True`` on the last micro-batch: groups reduce-scatter as soon as their backward completes."""
        self._sync_enabled = bool(enable)
        if enable:
            if self.world > 1:
                self.shard_comm.begin_grad_sync()
            for g in self.groups:
                g._pending = sum(1 for s in g.slots if s.param.requires_grad)
                g._reduced = False
                g._ready = False
            # Reductions are issued in ONE order on every rank: last block first (the order backward completes them), root
            # group last.  A group whose hooks have all fired waits until every group ahead of it in this order has been
            # issued; whatever is left (parameters that got no gradient on this rank: experts without tokens, a skipped
            # micro-batch) is issued in the same order by ``finish_grad_sync``.  The n-th collective of a step therefore
            # pairs the same group on all ranks no matter which parameters received gradients where.
            self._schedule = [g for g in reversed(self.groups) if g.trainable]
            self._cursor = 0

    def _drain_schedule(self, force: bool = False, before: Optional[FlatGroup] = None) -> None:
        """Issue the reductions of all groups at the head of the schedule that are ready (``force``: ready or not), stopping
        in front of ``before`` when given."""
        sched = self._schedule
        if sched is None:
            return
        while self._cursor < len(sched):
            g = sched[self._cursor]
            if g is before or not (force or getattr(g, "_ready", False)):
                break
            if not getattr(g, "_reduced", False):
                g.ensure_grad_buffers()
                self._launch_reduce(g)
            self._cursor += 1

    def _launch_reduce(self, g: FlatGroup) -> None:
        if g.expert_local:  # the gradient already sums over every rank's tokens: match the rank-averaged objective
            g.main_grad.div_(float(self.world))
            g._reduced = True
            return
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                self.shard_comm.reduce_scatter_grad(g)
        else:
            self.shard_comm.reduce_scatter_grad(g)
        if self.replicate_comm is not None:
            if self._comm_stream is not None:
                with torch.cuda.stream(self._comm_stream):
                    self.replicate_comm.all_reduce(g.grad_shard)
                    g.grad_shard.div_(self.replicate_comm.size)
            else:
                self.replicate_comm.all_reduce(g.grad_shard)
                g.grad_shard.div_(self.replicate_comm.size)
        g._reduced = True

    def finish_grad_sync(self) -> None:
        """Reduce any group whose hooks did not all fire (unused params) and join the comm stream."""
        if self.world > 1:
            if self._schedule is None:
                self.set_grad_sync(True)
            self._drain_schedule(force=True)
            if self._comm_stream is not None:
                torch.cuda.current_stream().wait_stream(self._comm_stream)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (averaged) gradient as a device scalar."""
        fused = self.shard_comm.local_sumsq() if self.world > 1 else None
        if fused is not None:
            total = fused.clone().reshape(1)
            for g in self.groups:
                if g.expert_local and g.trainable and g.grad_shard is not None:
                    total = total + O.sum_squares(g.grad_shard).reshape(1)
        else:
            parts = [O.sum_squares(g.grad_shard) for g in self.groups if g.trainable and g.grad_shard is not None]
            total = torch.stack(parts).sum() if parts else torch.zeros((), device=self.device)
            total = total.reshape(1).float()
        self.comm.all_reduce(total)
        return total.sqrt().reshape(()) * float(self.grad_replicas)

    def optimizer_step(self, *, lr: float, betas: Tuple[float, float], eps: float, weight_decay: float, step: int,
                       clip_coef: Optional[torch.Tensor] = None, ema_decay: Optional[float] = None) -> None:
        for g in self.groups:
            if not g.trainable or g.grad_shard is None:
                continue
            if self.grad_replicas > 1:
                g.grad_shard.mul_(float(self.grad_replicas))
            if g.expert_local:
                O.adamw_step(g.master, g.grad_shard, g.exp_avg, g.exp_avg_sq, lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay,
                             step=step, low=g.param_shard, ema=g.ema if ema_decay is not None else None, ema_decay=ema_decay or 0.0, grad_scale_tensor=clip_coef)
                continue
            if self.world > 1 and self.shard_comm.fused_optimizer:
                self.shard_comm.adamw_publish(g, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, step=step, clip_coef=clip_coef,
                                              ema=g.ema if ema_decay is not None else None, ema_decay=ema_decay or 0.0)
                continue
            released = not g._gathered
            O.adamw_step(g.master, g.grad_shard, g.exp_avg, g.exp_avg_sq, lr=lr, beta1=betas[0], beta2=betas[1], eps=eps,
                         weight_decay=weight_decay, step=step, low=g.shard_resident if released else g.param_shard,
                         ema=g.ema if ema_decay is not None else None, ema_decay=ema_decay or 0.0, grad_scale_tensor=clip_coef)
            if not released:  # a released replica is rebuilt from the shards at its next use
                self.shard_comm.publish_params(g)

    def release_grad_buffers(self) -> None:
        for g in self.groups:
            g.release_grad_buffers()

    # ---- state -----------------------------------------------------------------------------------------
    def named_full_params(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for g in self.groups:
            for s in g.slots:
                yield s.name, s.param.data

    def sync_master_from_params(self) -> None:
        """After loading weights into the bf16 views: refresh the fp32 master shards."""
        for g in self.groups:
            g.master.copy_(g.param_shard.to(g.master_dtype))

    def optimizer_state_dict(self) -> Dict[str, Any]:
        """Full (gathered) optimizer state keyed by parameter NAME, each entry ``{master, exp_avg, exp_avg_sq}`` — the checkpoint
        key ``optimizer_state_dict`` is the reference's, the layout under it is this runtime's (a ``torch.optim.AdamW`` state dict
        is keyed by integer index and has no fp32 master).  Parameters owned by one expert-parallel rank are not gathered: every
        rank's copy is kept under ``<name>#ep<rank>``."""
        out: Dict[str, Any] = {}
        for g in self.groups:
            if g.expert_local:
                mine = {s.name: {k: getattr(g, k).float()[s.offset : s.offset + s.numel].view(s.shape).cpu().clone()
                                 for k in ("master", "exp_avg", "exp_avg_sq")} for s in g.slots}
                per_rank = self.comm.all_gather_object(mine) if self.comm.active else [mine]
                for r, d in enumerate(per_rank):
                    for name, st in d.items():
                        out[f"{name}#ep{r}"] = st
                continue
            full = {}
            for key in ("master", "exp_avg", "exp_avg_sq"):
                t = getattr(g, key).float()
                full[key] = torch.cat(self.comm.all_gather(t)) if self.comm.active else t
            for s in g.slots:
                out[s.name] = {k: full[k][s.offset : s.offset + s.numel].view(s.shape).cpu().clone() for k in full}
        return out

    def load_optimizer_state_dict(self, sd: Dict[str, Any]) -> None:
        import logging

        matched = 0
        for g in self.groups:
            lo, hi = g.shard_range()
            suffix = f"#ep{self.rank}" if g.expert_local else ""
            for key in ("master", "exp_avg", "exp_avg_sq"):
                full = torch.zeros(g.padded, dtype=torch.float32)
                for s in g.slots:
                    entry = sd.get(s.name + suffix)
                    if isinstance(entry, dict) and key in entry:
                        full[s.offset : s.offset + s.numel] = entry[key].reshape(-1).float()
                        matched += 1
                    elif key == "master":
                        full[s.offset : s.offset + s.numel] = s.param.data.reshape(-1).float().cpu()
                getattr(g, key).copy_(full[lo:hi].to(getattr(g, key).dtype))
        if sd and not matched:
            logging.getLogger(__name__).warning(
                "load_optimizer_state_dict: none of the %d entries matches a parameter name of this model (an index-keyed "
                "torch.optim state dict?); moments start at zero and the master weights come from the loaded parameters", len(sd))

    def offload(self) -> None:
        """Move optimizer shards to pinned host memory (colocated rollout needs the HBM)."""
        for g in self.groups:
            for key in ("master", "exp_avg", "exp_avg_sq"):
                t = getattr(g, key)
                if t.device.type == "cuda":
                    host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                    host.copy_(t, non_blocking=True)
                    setattr(g, key, host)
            g.release_grad_buffers()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()

    def onload(self) -> None:
        for g in self.groups:
            for key in ("master", "exp_avg", "exp_avg_sq"):
                t = getattr(g, key)
                if t.device != self.device:
                    setattr(g, key, t.to(self.device, non_blocking=True))

    def state_bytes(self) -> int:
        return sum(g.state_bytes() for g in self.groups)


__all__ = ["FlatShardedModel", "FlatGroup", "ShardComm", "ParamSlot", "ALIGN"]
