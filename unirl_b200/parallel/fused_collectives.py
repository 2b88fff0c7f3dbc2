"""Peer-memory collectives fused with their compute step (NVLink P2P loads/stores inside our own kernels).

Plumbing: torch symmetric memory provides one allocation per rank whose peers' addresses are mapped into
this process (``buffer_ptrs``).  A :class:`PeerArena` is such an allocation plus a tiny symmetric flag pad
and a local state word block; the kernels in ``csrc/peer.cu`` rendezvous through the flags (bounded waits,
status word instead of a trap) and move data with plain vector loads/stores on the peers' addresses.

What is fused
-------------
``FusedAllReduce``   TP row-parallel projection → *one* kernel that sums the partial outputs of all TP ranks,
                     adds the residual and applies the next RMSNorm.  The projection GEMM writes its output
                     straight into the symmetric staging buffer, so the partial never makes an extra trip.
``FusedShardComm``   sharded trainer: gradient reduce-scatter that also averages and accumulates the squared
                     norm of the result (one kernel, pull from peers); AdamW whose bf16 output is stored into
                     every rank's parameter replica (update + all-gather in one kernel).
``reshard_scatter_local``  trainer replica → rollout-engine TP shards, all parameters in ONE launch driven by a
                     device-resident copy table.

NCCL remains the fallback (and the measured baseline) whenever symmetric memory cannot be set up.
Reference behaviour replaced: FSDP2 reduce-scatter / all-gather (``unirl/train/inject.py:189-383``), clip
(``unirl/train/fsdp_utils.py:274-319``), bucketed weight broadcast (``unirl/distributed/weight_sync/full/nccl.py:142-181``).
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.ops import _ext
from unirl_b200.parallel.flat_shard import FlatGroup, ShardComm

logger = logging.getLogger(__name__)

_FLAG_WORDS = 64  # 4 slots x 8 peers, padded


class PeerCommError(RuntimeError):
    """A bounded device-side wait for a peer ran out of time (code = 300 + 10·kernel + peer rank)."""


def peer_memory_available(comm: Optional[Comm], device: Any) -> bool:
    dev = torch.device(device)
    return bool(comm is not None and comm.active and comm.size <= 8 and dev.type == "cuda" and _ext.have_ext())


class PeerArena:
    """One symmetric allocation (``nbytes`` per rank) + flag pad + device state, bound to a ``_C.PeerComm``."""

    def __init__(self, comm: Comm, nbytes: int, device: Any, wait_s: float = 20.0):
        import torch.distributed._symmetric_memory as symm

        C = _ext.require_ext()
        self.comm, self.device = comm, torch.device(device)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        group = comm.group
        name = getattr(group, "group_name", None) or group
        self._buf = symm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self._hdl = symm.rendezvous(self._buf, group=name)
        self._flag_t = symm.empty(_FLAG_WORDS, dtype=torch.int32, device=self.device)
        self._flag_t.zero_()
        self._flag_h = symm.rendezvous(self._flag_t, group=name)
        self.state = torch.zeros(8, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        comm.barrier()  # every pad is zero before anyone signals
        self.rank, self.world = comm.rank, comm.size
        self.peer = C.PeerComm([int(p) for p in self._hdl.buffer_ptrs], [int(p) for p in self._flag_h.buffer_ptrs], self.rank, self.state, float(wait_s))
        self._cursor = 0
        from unirl_b200.ops.status import register_checker

        register_checker(self)  # status word read at every step boundary (check_device_status)

    def take(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Bump-allocate a zeroed 256-byte aligned view of this rank's part of the arena."""
        size = numel * torch.empty((), dtype=dtype).element_size()
        start = (self._cursor + 255) // 256 * 256
        if start + size > self.nbytes:
            raise MemoryError(f"PeerArena exhausted: need {start + size} of {self.nbytes} bytes")
        self._cursor = start + size
        return self._buf[start : start + size].view(dtype).zero_()

    def check(self) -> None:
        """Host read of the status word (synchronises); raises if any wait timed out since the last check."""
        code = int(self.state[4].item())
        if code:
            self.state[4].zero_()
            raise PeerCommError(f"peer wait timed out on rank {self.rank} (code {code}: kernel {(code - 300) // 10}, peer {code % 10 if code % 10 < 5 else code % 10 - 5})")

    def barrier(self) -> None:
        _ext.require_ext().peer_barrier(self.peer)
        _ext.count_launch()


# ------------------------------------------------------------------------------------------------ TP all-reduce
class FusedAllReduce:
    """``x_new = residual + Σ_ranks (inp @ W_rankᵀ)``, ``h = RMSNorm(x_new)·w`` with one GEMM and one peer kernel.

    Two staging halves alternate call by call (a peer may still be reading the previous half while this rank's
    next GEMM runs).  A sequence that is replayed (CUDA graph) must start and end on half 0 with a rendezvous in
    between — :meth:`align` enforces that and is cheap when already aligned.
    """

    def __init__(self, comm: Comm, max_tokens: int, hidden: int, device: Any, wait_s: float = 20.0):
        import os

        self.max_tokens, self.hidden = int(max_tokens), int(hidden)
        # decode-sized projections run GEMM + all-reduce as ONE kernel: every rank's epilogue stores its partial tile into every peer
        # (slot per source rank, two halves alternating with the epoch) and sums the peers' tiles once their per-CTA flags arrive.
        # Up to one 128-row tile by default: at 256 rows (two tiles re-reading the weights) GEMM + separate peer kernel measured faster
        # (5.82 vs 6.37 ms per 36-layer decode step at TP=2, batch 256); UNIRL_B200_TP_FUSED_GEMM_MAX_M widens it.
        self.fused_rows = int(os.environ.get("UNIRL_B200_TP_FUSED_GEMM_MAX_M", "128")) if os.environ.get("UNIRL_B200_TP_FUSED_GEMM", "1") == "1" else 0
        self.fused_rows = min(self.fused_rows, self.max_tokens)
        world = comm.size
        slot = self.fused_rows * self.hidden
        extra = (2 * world * slot * 2 + world * 1024 * 4 + 1024) if self.fused_rows else 0
        self.arena = PeerArena(comm, 2 * self.max_tokens * self.hidden * 2 + 512 + extra, device, wait_s)
        self._halves = [self.arena.take(self.max_tokens * self.hidden, torch.bfloat16) for _ in range(2)]
        self._gemm_stage = self.arena.take(2 * world * slot, torch.bfloat16) if self.fused_rows else None
        self._gemm_flags = self.arena.take(world * 1024, torch.int32) if self.fused_rows else None
        if self.fused_rows:
            torch.cuda.synchronize(device)
            comm.barrier()  # every rank's flag area is zero before any peer publishes into it
        self.fused_calls = 0
        self._half = 0
        self._C = _ext.require_ext()
        self.comm = comm

    def align(self) -> None:
        if self._half != 0:
            self.arena.barrier()
            self._half = 0

    def _stage(self, T: int) -> torch.Tensor:
        buf = self._halves[self._half][: T * self.hidden].view(T, self.hidden)
        self._half ^= 1
        return buf

    def proj_reduce_norm(self, inp: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor],
                         eps: float) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        T = inp.shape[0]
        if T > self.max_tokens:  # oversize batch: library collective
            y = torch.matmul(inp, weight.t())
            self.comm.all_reduce(y)
            x = y if residual is None else y + residual
            from unirl_b200.ops.norm import rmsnorm

            return x, (rmsnorm(x, norm_weight, eps) if norm_weight is not None else None)
        if (0 < T <= self.fused_rows and inp.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and inp.shape[1] % 64 == 0 and weight.shape[0] == self.hidden
                and self.hidden % 8 == 0 and self.hidden >= 1024 and weight.is_contiguous() and hasattr(self._C, "gemm_skinny_allreduce")):
            x = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=inp.device)
            self._C.gemm_skinny_allreduce(self.arena.peer, self._gemm_stage, self._gemm_flags, inp.contiguous(), weight,
                                          residual.contiguous() if residual is not None else None, x)
            _ext.count_launch()
            self.fused_calls += 1
            if norm_weight is None:
                return x, None
            from unirl_b200.ops.norm import rmsnorm

            return x, rmsnorm(x, norm_weight, eps)
        part = self._stage(T)
        from unirl_b200.ops.linear import skinny_linear

        if skinny_linear(inp, weight, None, out=part) is None:
            torch.matmul(inp, weight.t(), out=part)
        x = torch.empty_like(part)
        h = torch.empty_like(part) if norm_weight is not None else None
        self._C.peer_allreduce_residual_rmsnorm(self.arena.peer, part, residual, norm_weight, x, h, float(eps))
        _ext.count_launch()
        return x, h

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        """Plain all-reduce of an existing tensor (copied through the staging half)."""
        T = y.numel() // self.hidden
        if y.dtype != torch.bfloat16 or y.numel() % self.hidden or T > self.max_tokens:
            return self.comm.all_reduce(y)
        part = self._stage(T)
        part.copy_(y.reshape(T, self.hidden))
        out = torch.empty_like(part)
        self._C.peer_allreduce_residual_rmsnorm(self.arena.peer, part, None, None, out, None, 0.0)
        _ext.count_launch()
        return out.view_as(y)


def make_fused_all_reduce(comm: Comm, max_tokens: int = 16384, hidden: int = 0, device: Any = None) -> Optional[FusedAllReduce]:
    device = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
    if not peer_memory_available(comm, device) or hidden <= 0:
        return None
    return FusedAllReduce(comm, max_tokens, hidden, device)


# ------------------------------------------------------------------------------------------------ Ulysses exchange
class FusedUlyssesExchange:
    """Sequence-shard ↔ head-shard exchange of the Ulysses attention through peer memory: the activation is staged once in
    this rank's symmetric arena and ONE kernel on every rank pulls its slice from all peers, writing it already permuted
    (the library path packs, runs an all-to-all and unpacks: three passes and two extra buffers).  Differentiable: the
    backward of one direction is the other direction."""

    def __init__(self, comm: Comm, device: Any, wait_s: float = 60.0):
        self.comm, self.device, self.wait_s = comm, torch.device(device), float(wait_s)
        self.arena: Optional[PeerArena] = None
        self._stage: Optional[torch.Tensor] = None
        self._C = _ext.require_ext()

    def _staging(self, numel: int) -> torch.Tensor:
        if self._stage is None or self._stage.numel() < numel:  # collective and deterministic: every rank grows at the same call
            cap = max(numel, 1 << 20)
            self.arena = PeerArena(self.comm, cap * 2 + 512, self.device, self.wait_s)
            self._stage = self.arena.take(cap, torch.bfloat16)
        return self._stage[:numel]

    def exchange(self, x: torch.Tensor, mode: int) -> torch.Tensor:
        """``mode 0``: ``[B, l, P·Hp, D] → [B, P·l, Hp, D]``; ``mode 1``: ``[B, P·l, Hp, D] → [B, l, P·Hp, D]``."""
        p = self.comm.size
        if mode == 0:
            b, l, h, d = x.shape
            hp = h // p
        else:
            b, lp, hp, d = x.shape
            l = lp // p
        stage = self._staging(x.numel())
        stage.view(x.shape).copy_(x)
        out = self._C.peer_ulysses_exchange(self.arena.peer, stage, b, l, hp, d, mode)
        _ext.count_launch()
        return out

    def supports(self, x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0

    def check(self) -> None:
        if self.arena is not None:
            self.arena.check()


class _FusedExchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, ex: "FusedUlyssesExchange", mode: int) -> torch.Tensor:
        ctx.ex, ctx.mode = ex, mode
        return ex.exchange(x.contiguous(), mode)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        return ctx.ex.exchange(g.contiguous(), 1 - ctx.mode), None, None


def make_fused_ulysses_exchange(comm: Comm, device: Any = None) -> Optional[FusedUlyssesExchange]:
    device = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
    if not peer_memory_available(comm, device):
        return None
    return FusedUlyssesExchange(comm, device)


class FusedHeadScatterProjection:
    """QKV projection whose epilogue IS the sequence-shard → head-shard exchange: the tcgen05 GEMM stores every 64-column box of its
    output straight into the memory of the rank that owns the box's head, at the row this rank's tokens have in the gathered sequence
    (plain 16-byte stores on the symmetric mapping; no staging copy, no separate exchange pass).  One rendezvous kernel follows the GEMM;
    after it ``recv[part, b, p·l + t, hh, :]`` on rank ``r`` holds rank ``p``'s token ``t``, head ``r·Hp + hh`` of part (q, k, v).

    Two receive buffers alternate call by call: a peer may start the next projection's stores while this rank still reads the previous
    result, but never the one before it (every call ends in a rendezvous that all ranks enter only after consuming the older buffer).
    Columns past the routed parts (the MLP half of a fused single-stream projection) stay local and are returned as they are."""

    def __init__(self, comm: Comm, device: Any, wait_s: float = 60.0):
        self.comm, self.device, self.wait_s = comm, torch.device(device), float(wait_s)
        self.arena: Optional[PeerArena] = None
        self._recv: List[torch.Tensor] = []
        self._tables: Dict[Tuple, torch.Tensor] = {}
        self._flip = 0
        self.calls = 0
        self._C = _ext.require_ext()

    def _buffers(self, numel: int) -> None:
        if not self._recv or self._recv[0].numel() < numel:  # collective and deterministic: every rank grows at the same call
            cap = max(numel, 1 << 20)
            self.arena = PeerArena(self.comm, 2 * (cap * 2 + 256) + 512, self.device, self.wait_s)
            self._recv = [self.arena.take(cap, torch.bfloat16) for _ in range(2)]
            # `take` zeroes the views with a memset queued on THIS rank's stream.  A faster peer's projection may store into them as soon as
            # it has its own table, so every rank's memset must have run before any rank goes on (at 8 ranks a late memset wiped rows that a
            # peer had already delivered).
            torch.cuda.synchronize(self.device)
            self.comm.barrier()
            self._tables.clear()
            self._flip = 0

    @staticmethod
    def route_rows(peer_bases: Sequence[int], rank: int, world: int, B: int, l: int, heads: int, head_dim: int, parts: int, n_cols: int,
                   stat_parts: int = 0) -> List[Tuple[int, int, int, int]]:
        """Routing table rows ``(address, stride, extra, slot)`` per 64-column box for an output of ``n_cols`` columns laid out
        ``[parts x heads x head_dim | local columns]``; ``peer_bases[p]`` is the byte address of rank ``p``'s receive buffer.  The boxes of
        the first ``stat_parts`` parts also add their rows' sums of squares to statistic ``slot = part``."""
        hp = heads // world
        rows: List[Tuple[int, int, int, int]] = []
        for col in range(0, n_cols, 64):
            if col >= parts * heads * head_dim:
                rows.append((0, 0, 0, -1))
                continue
            part, rem = divmod(col, heads * head_dim)
            head, d0 = divmod(rem, head_dim)
            dst, hl = divmod(head, hp)
            elem = part * B * world * l * hp * head_dim + rank * l * hp * head_dim + hl * head_dim + d0
            rows.append((int(peer_bases[dst]) + 2 * elem, hp * head_dim, (world - 1) * l, part if part < stat_parts else -1))
        return rows

    @staticmethod
    def pack_table(rows: Sequence[Tuple[int, ...]], device: Any) -> torch.Tensor:
        """Rows ``(address, stride, extra[, slot])`` → the device table of 24-byte entries; ``slot`` (default -1: none) names the row-statistic a box adds to."""
        return torch.tensor([[r[0], r[1] | (r[2] << 32), (r[3] if len(r) > 3 else -1) & 0xFFFFFFFF] for r in rows], dtype=torch.int64).to(device)

    def supports(self, x: torch.Tensor, weight: torch.Tensor, heads: int, head_dim: int) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and head_dim % 64 == 0 and heads % self.comm.size == 0
                and weight.shape[0] % 64 == 0 and weight.shape[1] % 64 == 0 and x.dim() == 3 and hasattr(self._C, "gemm_bf16_route"))

    def project(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], heads: int, head_dim: int, parts: int = 3,
                stat_parts: int = 0) -> Tuple[torch.Tensor, ...]:
        """``x [B, l, K]`` → ``(recv [parts, B, P·l, Hp, D]`` — a view of a symmetric buffer that the call after next overwrites —, local columns or None)``;
        with ``stat_parts > 0`` a third item: ``[stat_parts, B, l]`` fp32, per token of THIS rank the sum of squares over all heads of each of the
        first ``stat_parts`` parts (what an RMS norm spanning the heads needs, gathered by the caller)."""
        world, rank = self.comm.size, self.comm.rank
        b, l, _ = x.shape
        hp, n = heads // world, weight.shape[0]
        numel = parts * b * world * l * hp * head_dim
        self._buffers(numel)
        buf = self._flip
        self._flip ^= 1
        key = (buf, b, l, heads, head_dim, parts, n, stat_parts)
        table = self._tables.get(key)
        if table is None:
            off = self._recv[buf].data_ptr() - self.arena._buf.data_ptr()
            bases = [int(pb) + off for pb in self.arena._hdl.buffer_ptrs]
            table = self.pack_table(self.route_rows(bases, rank, world, b, l, heads, head_dim, parts, n, stat_parts), x.device)
            self._tables[key] = table
        local_cols = n - parts * heads * head_dim
        rowsq = torch.zeros(stat_parts, b * l, dtype=torch.float32, device=x.device) if stat_parts else None
        rest = self._C.gemm_bf16_route(x.reshape(b * l, -1).contiguous(), weight, bias, table, l, local_cols, rowsq)
        _ext.count_launch()
        self.arena.barrier()  # every rank's stores into this rank's buffer have landed
        self.calls += 1
        out = self._recv[buf][:numel].view(parts, b, world * l, hp, head_dim)
        rest = rest.view(b, l, local_cols) if local_cols else None
        return (out, rest, rowsq.view(stat_parts, b, l)) if stat_parts else (out, rest)

    def align(self) -> None:
        """End a forward pass on buffer 0.  A pass with an odd number of projections would otherwise begin its next run (a replayed CUDA graph
        repeats the captured buffer order) on the buffer its last projection used, which a peer may still be reading: one more rendezvous
        makes every rank finish reading first."""
        if self._flip:
            self.arena.barrier()
            self._flip = 0

    def check(self) -> None:
        if self.arena is not None:
            self.arena.check()


def make_fused_head_scatter(comm: Comm, device: Any = None) -> Optional[FusedHeadScatterProjection]:
    device = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
    if not peer_memory_available(comm, device):
        return None
    return FusedHeadScatterProjection(comm, device)


# ------------------------------------------------------------------------------------------------ sharded trainer
class FusedShardComm(ShardComm):
    """Sharded-trainer collectives through peer memory: replicas and gradient buffers live in symmetric arenas."""

    fused_optimizer = True
    persistent_grads = True

    def __init__(self, comm: Comm, wait_s: float = 60.0):
        super().__init__(comm)
        if not _ext.have_ext():
            raise RuntimeError("native extension missing")
        self.wait_s = wait_s
        self.param_arena: Optional[PeerArena] = None
        self.grad_arena: Optional[PeerArena] = None
        self.norm_sq: Optional[torch.Tensor] = None
        self._C = _ext.require_ext()

    # -- allocation hooks used by FlatGroup ----------------------------------------------------------------
    def reserve(self, param_bytes: int, grad_bytes: int, device: Any) -> None:
        slack = 1 << 16
        self.param_arena = PeerArena(self.comm, param_bytes + slack, device, self.wait_s)
        self.grad_arena = PeerArena(self.comm, grad_bytes + slack, device, self.wait_s) if grad_bytes else None
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=device)

    def alloc_param(self, numel: int, dtype: torch.dtype, device: Any) -> torch.Tensor:
        return self.param_arena.take(numel, dtype)

    def alloc_grad(self, numel: int, device: Any) -> torch.Tensor:
        return self.grad_arena.take(numel, torch.float32)

    # -- collectives ----------------------------------------------------------------------------------------
    def begin_grad_sync(self) -> None:
        self.norm_sq.zero_()

    def reduce_scatter_grad(self, group: FlatGroup) -> None:
        self._C.peer_reduce_scatter_sumsq(self.grad_arena.peer, group.main_grad, group.grad_shard, self.norm_sq, 1.0 / self.comm.size)
        _ext.count_launch()

    def local_sumsq(self) -> torch.Tensor:
        return self.norm_sq

    def adamw_publish(self, group: FlatGroup, *, lr: float, betas: Tuple[float, float], eps: float, weight_decay: float, step: int,
                      clip_coef: Optional[torch.Tensor], ema: Optional[torch.Tensor], ema_decay: float) -> None:
        self._C.peer_adamw_publish(self.param_arena.peer, group.flat_param, group.master, group.grad_shard, group.exp_avg, group.exp_avg_sq, ema,
                                   float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay), int(step), clip_coef, float(ema_decay))
        _ext.count_launch()

    def publish_params(self, group: FlatGroup) -> None:  # folded into adamw_publish
        return None

    def check(self) -> None:
        for a in (self.param_arena, self.grad_arena):
            if a is not None:
                a.check()


# ------------------------------------------------------------------------------------------------ reshard
_TABLE_CACHE: Dict[int, Tuple[torch.Tensor, int, int, Any]] = {}


def build_copy_table(plan: Sequence[Tuple[torch.Tensor, torch.Tensor, Any]]) -> Tuple[torch.Tensor, int]:
    """``[(src_flat, dst_flat, CopyOp)]`` → int64 ``[n, 6]`` host table (src ptr, dst ptr, rows, row_len, strides) and the largest copy in 16-byte vectors."""
    rows: List[List[int]] = []
    max_vecs = 1
    for src, dst, op in plan:
        es = src.element_size()
        rows.append([src.data_ptr() + op.src_off * es, dst.data_ptr() + op.dst_off * es, op.rows, op.row_len, op.src_stride, op.dst_stride])
        max_vecs = max(max_vecs, op.rows * op.row_len // 8)
    return torch.tensor(rows, dtype=torch.int64).reshape(-1, 6), max_vecs


def reshard_scatter_local(plan: Sequence[Tuple[torch.Tensor, torch.Tensor, Any]]) -> bool:
    """Execute a copy plan (bf16 tensors on one CUDA device, destinations local or peer-mapped) in one kernel launch."""
    if not plan or not _ext.have_ext():
        return False
    src0 = plan[0][0]
    if not src0.is_cuda or any(s.dtype != torch.bfloat16 or d.dtype != torch.bfloat16 for s, d, _ in plan):
        return False
    key = id(plan)
    ent = _TABLE_CACHE.get(key)
    sig = (len(plan), plan[0][0].data_ptr(), plan[-1][1].data_ptr())
    if ent is None or ent[3] != sig:
        host, max_vecs = build_copy_table(plan)
        ent = (host.to(src0.device), len(plan), max_vecs, sig)
        _TABLE_CACHE[key] = ent
    _ext.require_ext().peer_scatter_copy(ent[0], ent[1], ent[2])
    _ext.count_launch()
    return True


__all__ = ["PeerArena", "PeerCommError", "FusedAllReduce", "make_fused_all_reduce", "FusedUlyssesExchange", "make_fused_ulysses_exchange", "FusedShardComm", "reshard_scatter_local", "build_copy_table",
           "peer_memory_available"]
