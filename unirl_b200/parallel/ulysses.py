"""Ulysses sequence parallelism for the DiT attention: ranks hold ``L / P`` latent tokens each; around the attention core
the sequence shards are exchanged for head shards (``[B, L/P, H, D] → [B, L, H/P, D]``) and back.

Text tokens of a joint block are replicated on every rank (they are few), so the exchange only moves the latent part:
after the first all-to-all every rank holds ALL latent tokens and ALL text tokens for ITS ``H / P`` heads, runs plain
attention, and the second all-to-all returns the latent outputs to their sequence owners; text outputs are all-gathered
over heads.

Collectives go through :class:`Comm` (NCCL all-to-all over NVLink; gloo emulation on CPU for tests).
Parity: the ``ulysses_degree`` knob the reference passes to its external engines
(``unirl/rollout/engine/vllm_omni/stage_configs/sd35_t2i_rl.yaml:42-54``, ``patch_denoising.py:137``) — here a first-class
part of the model code so the trainer uses it too.
"""

from __future__ import annotations

import os
from typing import Any, Optional

import torch

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.ops.attention import dense_attention


class _SeqToHead(torch.autograd.Function):
    """``[B, l, H, D]`` (sequence shard, all heads) → ``[B, l·P, H/P, D]`` (all tokens, head shard); backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm = comm
        return _a2a_seq_to_head(x, comm)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        return _a2a_head_to_seq(g.contiguous(), ctx.comm), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm = comm
        return _a2a_head_to_seq(x, comm)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        return _a2a_seq_to_head(g.contiguous(), ctx.comm), None


def _a2a_seq_to_head(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    p = comm.size
    b, l, h, d = x.shape
    send = x.view(b, l, p, h // p, d).permute(2, 0, 1, 3, 4).contiguous()  # [P(dst head group), B, l, H/P, D]
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send)  # recv[j] = rank j's tokens for my head group
    return recv.permute(1, 0, 2, 3, 4).reshape(b, p * l, h // p, d)


def _a2a_head_to_seq(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    p = comm.size
    b, lp, hp, d = x.shape
    l = lp // p
    send = x.view(b, p, l, hp, d).permute(1, 0, 2, 3, 4).contiguous()  # [P(dst seq owner), B, l, H/P, D]
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send)  # recv[j] = my tokens for rank j's head group
    return recv.permute(1, 2, 0, 3, 4).reshape(b, l, p * hp, d)


class _GatherHeads(torch.autograd.Function):
    """All-gather along the head axis (text outputs); backward keeps this rank's slice of the gradient (text is replicated,
    so every rank computes the same text gradient and no reduction is needed)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm, ctx.hp = comm, x.shape[2]
        parts = comm.all_gather(x.contiguous())
        return torch.cat(parts, 2)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        r = ctx.comm.rank
        return g[:, :, r * ctx.hp : (r + 1) * ctx.hp].contiguous(), None


class _ScatterProject(torch.autograd.Function):
    """``x [B, l, K]`` → ``[parts, B, P·l, H/P, D]``: the projection GEMM stores each head's columns into the owning rank's memory from its
    epilogue (forward).  Backward brings the gradient back with the head → sequence exchange and runs the two projection-gradient GEMMs."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], sp: "UlyssesContext", heads: int, head_dim: int, parts: int):
        out, rest = sp._scatter.project(x, weight, bias, heads, head_dim, parts)
        ctx.sp, ctx.parts, ctx.has_bias, ctx.has_rest = sp, parts, bias is not None, rest is not None
        if any(ctx.needs_input_grad[:3]):
            ctx.save_for_backward(x, weight)
            out = out.clone()  # the symmetric buffer is overwritten two calls later; what autograd keeps must not live there
        if rest is None:  # columns past the head parts (the MLP half of a single-stream block's one projection) stay on this rank
            rest = out.new_zeros(0)
            ctx.mark_non_differentiable(rest)
        return out, rest

    @staticmethod
    def backward(ctx, g: torch.Tensor, g_rest: Optional[torch.Tensor]):
        from unirl_b200.ops.linear import linear_grads

        x, weight = ctx.saved_tensors
        sp = ctx.sp
        b, l, _ = x.shape
        cols = [sp._exchange(g[i].contiguous(), 1).reshape(b * l, -1) for i in range(ctx.parts)]  # [B·l, H·D] each
        if ctx.has_rest:
            cols.append(g_rest.reshape(b * l, -1) if g_rest is not None else x.new_zeros(b * l, weight.shape[0] - sum(c.shape[1] for c in cols)))
        gy = torch.cat(cols, 1)
        gx, gw = linear_grads(gy, x.reshape(b * l, -1), weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        gb = gy.sum(0).to(weight.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return (gx.view_as(x) if gx is not None else None), gw, gb, None, None, None, None


class _ScatterProjectNormed(torch.autograd.Function):
    """:class:`_ScatterProject` followed by an RMS norm of q and k that spans ALL heads of a token (WAN), applied after the exchange.

    The norm's statistic — the sum of squares of a token's q (k) over every head — is accumulated by the projection's epilogue on the rank
    that owns the token and all-gathered (two floats per token); each rank then scales its own heads: ``q · rsqrt(ss / (H·D) + eps) · w``.
    Backward is the same norm's backward with the one cross-head reduction (``Σ_{h,d} g · w · q`` per token) summed over ranks."""

    @staticmethod
    def forward(ctx, x, weight, bias, wq, wk, sp: "UlyssesContext", heads: int, head_dim: int, eps: float):
        out, _, sq = sp._scatter.project(x, weight, bias, heads, head_dim, 3, stat_parts=2)
        ss = torch.cat(sp.comm.all_gather(sq.contiguous()), 2)  # [2, B, P·l]: rank p's tokens at p·l + t, like the exchanged sequence
        r = torch.rsqrt(ss / float(heads * head_dim) + eps)
        hp = heads // sp.size
        cols = slice(sp.rank * hp * head_dim, (sp.rank + 1) * hp * head_dim)
        q, k, v = out.unbind(0)
        qn = (q * r[0][..., None, None] * wq[cols].view(hp, head_dim).float()).to(q.dtype)
        kn = (k * r[1][..., None, None] * wk[cols].view(hp, head_dim).float()).to(k.dtype)
        ctx.sp, ctx.dims, ctx.has_bias = sp, (heads, head_dim, cols), bias is not None
        if any(ctx.needs_input_grad[:5]):
            ctx.save_for_backward(x, weight, q.clone(), k.clone(), r, wq, wk)
            v = v.clone()  # the symmetric buffer is overwritten two calls later
        return qn, kn, v

    @staticmethod
    def backward(ctx, gq: torch.Tensor, gk: torch.Tensor, gv: torch.Tensor):
        from unirl_b200.ops.linear import linear_grads

        x, weight, q, k, r, wq, wk = ctx.saved_tensors
        sp = ctx.sp
        heads, head_dim, cols = ctx.dims
        hp = heads // sp.size
        t, z, gw = [], [], []
        for g, raw, rr, w in ((gq, q, r[0], wq), (gk, k, r[1], wk)):
            g32, z32 = g.float(), raw.float()
            gw.append(torch.zeros_like(w, dtype=torch.float32).index_put_((torch.arange(cols.start, cols.stop, device=w.device),),
                                                                         (g32 * z32 * rr[..., None, None]).sum((0, 1)).flatten()).to(w.dtype))
            t.append(g32 * w[cols].view(hp, head_dim).float())
            z.append(z32)
        dr = sp.comm.all_reduce(torch.stack([(t[0] * z[0]).sum((-1, -2)), (t[1] * z[1]).sum((-1, -2))]))  # [2, B, P·l], summed over the ranks' heads
        dss = dr * (-0.5) * r.pow(3) / float(heads * head_dim)
        graw = [(t[i] * r[i][..., None, None] + 2.0 * z[i] * dss[i][..., None, None]).to(x.dtype) for i in range(2)]
        b, l, _ = x.shape
        gy = torch.cat([sp._exchange(g.contiguous(), 1).reshape(b * l, -1) for g in (graw[0], graw[1], gv)], 1)
        gx, gwt = linear_grads(gy, x.reshape(b * l, -1), weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        gb = gy.sum(0).to(weight.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return (gx.view_as(x) if gx is not None else None), gwt, gb, gw[0], gw[1], None, None, None, None


class UlyssesContext:
    def __init__(self, comm: Comm, collectives: str = "fused"):
        self.comm = comm
        self.size, self.rank = comm.size, max(comm.rank, 0)
        self.collectives = collectives  # fused (peer-memory exchange kernel) | nccl (pack + all-to-all + unpack)
        self._fused: Any = None
        self._fused_tried = False
        self._scatter: Any = None  # FusedHeadScatterProjection: the exchange inside the QKV projection's epilogue
        self._scatter_tried = False
        self.fuse_projection = os.environ.get("UNIRL_B200_ULYSSES_FUSED_QKV", "1") == "1"
        # the variant for q / k norms that span all heads of a token (row statistics from the epilogue, norm after the exchange) is opt-in
        self.fuse_projection_norm_over_heads = os.environ.get("UNIRL_B200_ULYSSES_FUSED_QKV_NORM_OVER_HEADS", "0") == "1"

    # ---- projection + exchange in one kernel --------------------------------------------------------------------
    def can_scatter_project(self, x: torch.Tensor, weight: torch.Tensor, heads: int, head_dim: Optional[int] = None) -> bool:
        """True when the QKV projection of ``x [B, l, K]`` can run as the GEMM whose epilogue stores head tiles to their owners.
        ``head_dim``: given when the weight has more rows than ``3 · heads · head_dim`` (trailing columns that stay local)."""
        if not (self.fuse_projection and self.collectives == "fused" and self.size > 1 and x.dim() == 3):
            return False
        if not self._scatter_tried and x.is_cuda:
            self._scatter_tried = True
            try:
                from unirl_b200.parallel.fused_collectives import make_fused_head_scatter

                self._scatter = make_fused_head_scatter(self.comm, x.device)
            except Exception:  # noqa: BLE001  (no symmetric memory on this system: projection, then exchange)
                self._scatter = None
        if head_dim is None:
            if weight.shape[0] % (3 * heads):
                return False
            head_dim = weight.shape[0] // (3 * heads)
        return self._scatter is not None and weight.shape[0] >= 3 * heads * head_dim and self._scatter.supports(x, weight, heads, head_dim)

    def scatter_project_normed(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], wq: torch.Tensor, wk: torch.Tensor, heads: int,
                               eps: float):
        """As :meth:`scatter_project`, with the q / k RMS norm that spans all heads of a token applied after the exchange → ``(q, k, v)``."""
        return _ScatterProjectNormed.apply(x, weight, bias, wq, wk, self, heads, weight.shape[0] // (3 * heads), float(eps))

    def scatter_project(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], heads: int, head_dim: Optional[int] = None):
        """``x [B, l, K]`` (this rank's tokens) → ``[3, B, P·l, H/P, D]`` (all tokens, this rank's heads) in one GEMM + one rendezvous.
        With ``head_dim`` given and more weight rows than ``3 · heads · head_dim``: ``(that, local [B, l, rest])``."""
        out, rest = _ScatterProject.apply(x, weight, bias, self, heads, head_dim or weight.shape[0] // (3 * heads), 3)
        return out if head_dim is None else (out, rest)

    def _exchange(self, x: torch.Tensor, mode: int) -> torch.Tensor:
        """Sequence shard → head shard (``mode 0``) or back (``mode 1``), on the peer-memory kernel when the tensors allow it."""
        if self.collectives == "fused" and x.is_cuda and not self._fused_tried:
            self._fused_tried = True
            try:
                from unirl_b200.parallel.fused_collectives import make_fused_ulysses_exchange

                self._fused = make_fused_ulysses_exchange(self.comm, x.device)
            except Exception:  # noqa: BLE001  (no symmetric memory on this system: library path)
                self._fused = None
        if self._fused is not None and self._fused.supports(x):
            from unirl_b200.parallel.fused_collectives import _FusedExchange

            return _FusedExchange.apply(x, self._fused, mode)
        return (_SeqToHead if mode == 0 else _HeadToSeq).apply(x.contiguous(), self.comm)

    def end_forward(self) -> None:
        """Called by the model after its last block: leaves the projection's receive buffers in their starting order."""
        if self._scatter is not None and hasattr(self._scatter, "align"):
            self._scatter.align()

    # ---- sequence sharding of the latent stream ---------------------------------------------------------------
    def shard_sequence(self, x: torch.Tensor) -> torch.Tensor:
        l = x.shape[1]
        if l % self.size:
            raise ValueError(f"latent sequence of {l} tokens does not split over {self.size} sequence-parallel ranks")
        n = l // self.size
        return x[:, self.rank * n : (self.rank + 1) * n]

    def shard_rope(self, table: torch.Tensor, n_text: int) -> torch.Tensor:
        """Rotary table ``[n_text + L, D/2]`` → this rank's ``[n_text + L/P, D/2]`` (text rows kept whole)."""
        lat = table[n_text:]
        n = lat.shape[0] // self.size
        return torch.cat([table[:n_text], lat[self.rank * n : (self.rank + 1) * n]])

    def gather_sequence(self, x: torch.Tensor) -> torch.Tensor:
        return _GatherSeq.apply(x, self.comm)

    # ---- attention ----------------------------------------------------------------------------------------------
    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_text: int = 0) -> torch.Tensor:
        """``q, k, v [B, n_text + L/P, H, D]`` → attention output with the same layout."""
        p, hp = self.size, q.shape[2] // self.size
        if q.shape[2] % p:
            raise ValueError(f"{q.shape[2]} heads do not split over {p} sequence-parallel ranks")
        lat = [self._exchange(t[:, n_text:], 0) for t in (q, k, v)]
        if n_text:
            txt = [t[:, :n_text, self.rank * hp : (self.rank + 1) * hp] for t in (q, k, v)]
            qq, kk, vv = (torch.cat([a, b], 1) for a, b in zip(txt, lat))
        else:
            qq, kk, vv = lat
        return self.finish(dense_attention(qq, kk, vv), n_text)

    def finish(self, o: torch.Tensor, n_text: int = 0) -> torch.Tensor:
        """Attention output ``[B, n_text + L, H/P, D]`` (all tokens, this rank's heads) → ``[B, n_text + L/P, H, D]``."""
        out_lat = self._exchange(o[:, n_text:], 1)
        if not n_text:
            return out_lat
        return torch.cat([_GatherHeads.apply(o[:, :n_text], self.comm), out_lat], 1)


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm, ctx.n = comm, x.shape[1]
        return torch.cat(comm.all_gather(x.contiguous()), 1)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        r = ctx.comm.rank
        return g[:, r * ctx.n : (r + 1) * ctx.n].contiguous(), None


__all__ = ["UlyssesContext"]
