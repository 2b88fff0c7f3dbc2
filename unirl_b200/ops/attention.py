"""Attention ops (K2, K3): packed-varlen attention for training/prefill, paged-KV decode attention.

Layouts
-------
``q [T, Hq, D]``, ``k/v [T, Hkv, D]`` packed over sequences delimited by ``cu_seqlens`` (no padding).
Paged cache: ``k_cache / v_cache [num_pages, Hkv, page_size, D]`` — one (page, head) block is a
contiguous ``page_size·D`` slab, which is what the decode kernel streams with bulk copies.
``block_tables [B, max_pages]`` (int32) maps a sequence's logical page to a physical page;
``slot_mapping [T]`` gives ``page · page_size + offset`` for each newly written token.

CUDA tensors run on the native kernels; the PyTorch expressions below are the CPU path and oracle.
"""

from __future__ import annotations

import math
import os
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from unirl_b200.ops._ext import count_launch, require_ext, use_native


# --------------------------------------------------------------------------------------- varlen
def varlen_attention_reference(q, k, v, cu_seqlens, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    hq, hkv = q.shape[1], k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        if e == s:
            continue
        qi = q[s:e].transpose(0, 1).unsqueeze(0)
        ki = k[s:e].transpose(0, 1).repeat_interleave(hq // hkv, 0).unsqueeze(0)
        vi = v[s:e].transpose(0, 1).repeat_interleave(hq // hkv, 0).unsqueeze(0)
        o = F.scaled_dot_product_attention(qi, ki, vi, is_causal=causal, scale=scale)
        out[s:e] = o.squeeze(0).transpose(0, 1)
    return out


def _varlen_impl() -> str:
    """``native``: the tcgen05 flash-attention kernels of this package (forward and backward); ``library``: cuDNN / flash-attn.
    ``UNIRL_B200_VARLEN_ATTN`` selects (``auto`` = native)."""
    want = os.environ.get("UNIRL_B200_VARLEN_ATTN", "auto")
    if want == "library":
        return "library"
    C = require_ext()
    if hasattr(C, "attn_varlen_fwd") and hasattr(C, "attn_varlen_bwd"):
        return "native"
    if want == "native":
        raise RuntimeError("UNIRL_B200_VARLEN_ATTN=native but the extension has no attn_varlen_fwd / attn_varlen_bwd")
    return "library"


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """The kernels read ``[T, H, D]`` through TMA: heads and features dense, row stride a multiple of 8 elements, 16-byte aligned base.
    Views into a fused qkv buffer qualify as they are; anything else is copied."""
    if t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale):
        C = require_ext()
        q, k, v = _rows_ok(q), _rows_ok(k), _rows_ok(v)
        cu = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
        out, lse = C.attn_varlen_fwd(q, k, v, cu, int(max_seqlen), bool(causal), float(scale))
        count_launch()
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.cfg = (int(max_seqlen), bool(causal), float(scale))
        return out

    @staticmethod
    def backward(ctx, g_out):
        C = require_ext()
        q, k, v, out, lse, cu = ctx.saved_tensors
        max_seqlen, causal, scale = ctx.cfg
        dq, dk, dv = C.attn_varlen_bwd(_rows_ok(g_out), q, k, v, out, lse, cu, max_seqlen, causal, scale)
        count_launch(3)
        return dq, dk, dv, None, None, None, None


def _library_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale):
    from flash_attn import flash_attn_varlen_func

    cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
    return flash_attn_varlen_func(q, k, v, cu, cu, int(max_seqlen), int(max_seqlen), 0.0, softmax_scale=float(scale), causal=bool(causal))


_PAD_WASTE_LIMIT = 1.35  # padded rows per real row above which the packed kernel is used instead of the dense one


def _dense_sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float) -> torch.Tensor:
    """``[B, L, H, D]`` through the dense fused-attention library kernel (cuDNN's Blackwell flash attention)."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    with sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION]):
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=bool(causal), scale=float(scale),
                                           enable_gqa=q.shape[2] != k.shape[2])
    return o.transpose(1, 2)


def _padded_dense(q, k, v, lens: Sequence[int], causal: bool, scale: float) -> Optional[torch.Tensor]:
    """Packed sequences → one padded ``[B, Lmax]`` batch for the dense kernel (differentiable).  Padding sits at the END of every row:
    under a causal mask no real query sees it; without a mask this path is only taken when no padding is needed."""
    b, lmax, t = len(lens), max(lens), q.shape[0]
    if b * lmax == t:  # equal lengths: pure views
        return _dense_sdpa(q.view(b, lmax, *q.shape[1:]), k.view(b, lmax, *k.shape[1:]), v.view(b, lmax, *v.shape[1:]), causal, scale).reshape(t, *q.shape[1:])
    if not causal or b * lmax > _PAD_WASTE_LIMIT * t:
        return None
    dst = torch.cat([torch.arange(n) + i * lmax for i, n in enumerate(lens)]).to(q.device)
    pad = lambda x: x.new_zeros(b * lmax, *x.shape[1:]).index_copy(0, dst, x).view(b, lmax, *x.shape[1:])  # noqa: E731
    o = _dense_sdpa(pad(q), pad(k), pad(v), causal, scale)
    return o.reshape(b * lmax, *q.shape[1:]).index_select(0, dst)


def varlen_attention(q, k, v, cu_seqlens, max_seqlen: Optional[int] = None, causal: bool = True, scale: Optional[float] = None,
                     lens_host: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Self attention over packed sequences (GQA when ``Hq > Hkv``).  ``lens_host``: the sequence lengths as host integers when the
    caller has them (avoids a device read); they let near-uniform batches run on the dense library kernel."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if use_native(q):
        if q.dtype not in (torch.bfloat16, torch.float16):
            return varlen_attention_reference(q, k, v, cu_seqlens, causal, scale)
        if _varlen_impl() == "native" and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and q.shape[1] % k.shape[1] == 0:
            return _VarlenAttention.apply(q, k, v, cu_seqlens, int(max_seqlen or 0), causal, scale)
        if lens_host is not None and os.environ.get("UNIRL_B200_DENSE_ATTN", "1") == "1" and q.shape[-1] in (64, 128):
            out = _padded_dense(q, k, v, [int(n) for n in lens_host], causal, scale)
            if out is not None:
                return out
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        return _library_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale)
    return varlen_attention_reference(q, k, v, cu_seqlens, causal, scale)


# --------------------------------------------------------------------------------------- paged KV
def kv_cache_write(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Scatter new ``k/v [T, Hkv, D]`` rows into the paged cache."""
    if use_native(k):
        require_ext().kv_cache_write(k.contiguous(), v.contiguous(), k_cache, v_cache, slot_mapping.to(torch.int64))
        count_launch()
        return
    page_size = k_cache.shape[2]
    page, off = slot_mapping // page_size, slot_mapping % page_size
    k_cache[page, :, off] = k
    v_cache[page, :, off] = v


def paged_decode_attention_reference(q, k_cache, v_cache, block_tables, seq_lens, scale: Optional[float] = None) -> torch.Tensor:
    b, hq, d = q.shape
    hkv, page_size = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    for i in range(b):
        n = int(seq_lens[i])
        pages = block_tables[i, : (n + page_size - 1) // page_size].long()
        kk = k_cache[pages].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n].float()
        vv = v_cache[pages].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n].float()
        qi = q[i].float().view(hkv, hq // hkv, d)
        p = torch.softmax(torch.einsum("hgd,hnd->hgn", qi, kk) * scale, -1)
        out[i] = torch.einsum("hgn,hnd->hgd", p, vv).reshape(hq, d).to(q.dtype)
    return out


def paged_decode_attention(q, k_cache, v_cache, block_tables, seq_lens, scale: Optional[float] = None,
                           workspace: Optional[torch.Tensor] = None, max_seq_len: Optional[int] = None) -> torch.Tensor:
    """One query token per sequence against its paged KV (split-KV + merge on CUDA).

    ``workspace`` (fp32) holds the split partials so a captured CUDA graph allocates nothing.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if use_native(q) and q.dtype == torch.bfloat16:
        out = require_ext().paged_decode_attention(q.contiguous(), k_cache, v_cache, block_tables, seq_lens, float(scale), workspace,
                                                   int(max_seq_len or 0))
        count_launch(2)
        return out
    return paged_decode_attention_reference(q, k_cache, v_cache, block_tables, seq_lens, scale)


def paged_decode_attention_cascade(q, k_cache, v_cache, cascade, scale: Optional[float] = None, workspace: Optional[torch.Tensor] = None,
                                   max_seq_len: Optional[int] = None) -> torch.Tensor:
    """Decode attention for batches in which groups of ``cascade.rows`` consecutive sequences share their leading KV pages (samples of one
    prompt): the shared prefix is read ONCE per group with the group's query heads stacked into one tile, every sequence's own suffix is
    read separately, and the two partial results are merged by their log-sum-exp.  ``cascade`` carries ``prefix_tables [B/R, Pp]``,
    ``prefix_lens [B/R]``, ``suffix_tables [B, Ps]``, ``suffix_lens [B]`` (int32) and ``rows``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    out = require_ext().paged_decode_attention_cascade(q.contiguous(), k_cache, v_cache, cascade.prefix_tables, cascade.prefix_lens, cascade.suffix_tables,
                                                       cascade.suffix_lens, int(cascade.rows), float(scale), workspace, int(max_seq_len or 0))
    count_launch(2)
    return out


# --------------------------------------------------------------------------------------- dense (DiT)
def dense_attention(q, k, v, scale: Optional[float] = None) -> torch.Tensor:
    """Bidirectional attention over ``[B, L, H, D]`` (joint text+image streams of MMDiT / video DiT).

    Routed through the packed kernel with uniform ``cu_seqlens`` on CUDA.
    """
    b, l, h, d = q.shape
    if use_native(q):
        if q.dtype in (torch.bfloat16, torch.float16) and d in (64, 128) and _varlen_impl() != "native" and os.environ.get("UNIRL_B200_DENSE_ATTN", "1") == "1":
            return _dense_sdpa(q, k, v, False, scale if scale is not None else 1.0 / math.sqrt(d))
        cu = torch.arange(0, (b + 1) * l, l, device=q.device, dtype=torch.int32)
        o = varlen_attention(q.reshape(b * l, h, d), k.reshape(b * l, k.shape[2], d), v.reshape(b * l, v.shape[2], d), cu, l, False, scale)
        return o.view(b, l, h, d)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=scale, enable_gqa=k.shape[2] != h)
    return o.transpose(1, 2)


__all__ = ["paged_decode_attention_cascade", "varlen_attention", "varlen_attention_reference", "kv_cache_write", "paged_decode_attention",
           "paged_decode_attention_reference", "dense_attention"]
