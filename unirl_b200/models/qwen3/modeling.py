"""Native Qwen3-style decoder (dense, GQA, QK-norm, SwiGLU) over *packed* token streams.

One module tree serves three execution modes through :class:`AttnMeta`:

* ``train``   – packed varlen causal attention with autograd (replay / log-prob recompute)
* ``prefill`` – same attention, additionally scatters K/V into the paged cache
* ``decode``  – one token per sequence against the paged cache (CUDA-graph friendly: no host syncs,
  all shapes static for a given batch size)

Parameters are stored *fused* — ``qkv_proj [(Hq+2Hkv)·D, H]`` and ``gate_up_proj [2I, H]`` — because that
is the layout the GEMM kernels want and it makes trainer→rollout weight sync a flat copy;
``hf_state_dict`` / ``load_hf_state_dict`` translate to the Hugging Face key grammar
(``model.layers.N.self_attn.q_proj.weight`` …) so checkpoints stay interchangeable.

Tensor parallelism (rollout engine): column-parallel ``qkv``/``gate_up``, row-parallel ``o``/``down``
followed by ``tp.all_reduce`` — the hook the fused GEMM→reduce kernels plug into.

The reference runs the Hugging Face ``Qwen3ForCausalLM`` re-padded to ``[B, L]``
(``unirl/models/qwen3/ar.py:330-447``); here nothing is ever padded.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from unirl_b200.ops import attention as A
from unirl_b200.ops.activation import swiglu
from unirl_b200.ops.linear import linear, linear_swiglu
from unirl_b200.ops.norm import add_rmsnorm, rmsnorm
from unirl_b200.ops.rope import qk_norm_rope
from unirl_b200.train.inject import lora_apply


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 2560
    intermediate_size: int = 9728
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    qk_norm: bool = True
    attention_bias: bool = False
    max_position_embeddings: int = 40960
    eos_token_id: int = 151643
    pad_token_id: int = 151643

    @classmethod
    def qwen3_4b(cls) -> "Qwen3Config":
        return cls()

    @classmethod
    def tiny(cls, **kw: Any) -> "Qwen3Config":
        base = dict(vocab_size=4096, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=64, eos_token_id=2, pad_token_id=0)
        base.update(kw)
        return cls(**base)

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        if "rope_theta" not in kw and isinstance(rope, dict) and rope.get("rope_theta") is not None:
            kw["rope_theta"] = float(rope["rope_theta"])  # newer config files nest the rotary base
        if "head_dim" not in kw:
            kw["head_dim"] = kw["hidden_size"] // kw["num_attention_heads"]
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        return cls(**kw)

    def num_params(self) -> int:
        h, i, d = self.hidden_size, self.intermediate_size, self.head_dim
        per_layer = h * (self.num_attention_heads + 2 * self.num_key_value_heads) * d + self.num_attention_heads * d * h + 3 * h * i + 2 * h + 2 * d
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return per_layer * self.num_hidden_layers + emb + h


@dataclass
class TPContext:
    """Tensor-parallel context of one rank: ``all_reduce`` sums partial row-parallel outputs."""

    rank: int = 0
    size: int = 1
    all_reduce: Optional[Callable[[torch.Tensor], torch.Tensor]] = None
    fused: Optional[Any] = None  # object with proj_reduce_norm(inp, weight, residual, norm_weight, eps) -> (x, h): GEMM + reduce + add + norm

    def reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.size == 1 or self.all_reduce is None else self.all_reduce(x)


@dataclass
class AttnMeta:
    mode: str = "train"  # train | prefill | decode
    positions: Optional[torch.Tensor] = None  # [T]
    cu_seqlens: Optional[torch.Tensor] = None  # [B+1] int32 on device
    max_seqlen: int = 0
    k_cache: Optional[List[torch.Tensor]] = None  # per layer [pages, Hkv, page, D]
    v_cache: Optional[List[torch.Tensor]] = None
    block_tables: Optional[torch.Tensor] = None  # [B, max_pages] int32
    seq_lens: Optional[torch.Tensor] = None  # [B] int32 (length INCLUDING the current token for decode)
    slot_mapping: Optional[torch.Tensor] = None  # [T] int64
    workspace: Optional[torch.Tensor] = None
    max_kv_len: int = 0
    cascade: Optional[Any] = None  # shared-prefix decode: prefix_tables / prefix_lens / suffix_tables / suffix_lens / rows
    seq_lens_host: Optional[List[int]] = None  # packed sequence lengths as host ints (saves a device read in attention dispatch)
    input_embeds: Optional[torch.Tensor] = None  # [T, H]: replaces the token-embedding lookup (multimodal prompts)
    cp_plan: Optional[Any] = None  # context parallelism: the packed stream holds this rank's chunk of every sequence (parallel.context_parallel.PackedPlan)
    cp_comm: Optional[Any] = None  # ... and the group its keys / values are gathered over


class Qwen3DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config, layer_idx: int, tp: TPContext, dtype: torch.dtype, device: Any):
        super().__init__()
        self.cfg, self.layer_idx, self.tp = cfg, layer_idx, tp
        if cfg.num_attention_heads % tp.size or cfg.num_key_value_heads % tp.size or cfg.intermediate_size % tp.size:
            raise ValueError(f"tp={tp.size} must divide heads ({cfg.num_attention_heads}/{cfg.num_key_value_heads}) and intermediate size")
        self.n_q, self.n_kv = cfg.num_attention_heads // tp.size, cfg.num_key_value_heads // tp.size
        self.inter = cfg.intermediate_size // tp.size
        d, h = cfg.head_dim, cfg.hidden_size
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))  # noqa: E731
        self.input_layernorm = mk(h)
        self.qkv_proj = mk((self.n_q + 2 * self.n_kv) * d, h)
        self.qkv_bias = mk((self.n_q + 2 * self.n_kv) * d) if cfg.attention_bias else None
        self.q_norm = mk(d) if cfg.qk_norm else None
        self.k_norm = mk(d) if cfg.qk_norm else None
        self.o_proj = mk(h, self.n_q * d)
        self.post_attention_layernorm = mk(h)
        self.gate_up_proj = mk(2 * self.inter, h)
        self.down_proj = mk(h, self.inter)
        self.scale = 1.0 / math.sqrt(d)

    def lora_targets(self) -> Dict[str, Tuple[str, int, int]]:
        d, nq, nkv, i = self.cfg.head_dim, self.n_q, self.n_kv, self.inter
        return {"q_proj": ("qkv_proj", 0, nq * d), "k_proj": ("qkv_proj", nq * d, nkv * d), "v_proj": ("qkv_proj", (nq + nkv) * d, nkv * d),
                "o_proj": ("o_proj", 0, self.cfg.hidden_size), "gate_proj": ("gate_up_proj", 0, i), "up_proj": ("gate_up_proj", i, i),
                "down_proj": ("down_proj", 0, self.cfg.hidden_size)}

    def hf_module_path(self, target: str) -> str:
        return f"model.layers.{self.layer_idx}.{'self_attn' if target in ('q_proj', 'k_proj', 'v_proj', 'o_proj') else 'mlp'}.{target}"

    def _proj(self, x: torch.Tensor, name: str, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if getattr(self, "_lora_index", None):
            y = lora_apply(self, name, x, linear(x, getattr(self, name)))
            return y if residual is None else y + residual
        return linear(x, getattr(self, name), residual=residual)

    def _gate_up_act(self, h: torch.Tensor) -> torch.Tensor:
        """``silu(h·Wgᵀ) ⊙ (h·Wuᵀ)``; without adapters the activation rides in the GEMM epilogue on decode-sized batches."""
        if getattr(self, "_lora_index", None):
            return swiglu(self._proj(h, "gate_up_proj"))
        return linear_swiglu(h, self.gate_up_proj)

    def _qkv_rope(self, h: torch.Tensor, meta: AttnMeta) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Fused QKV projection (+ bias) → per-head RMS q/k norm → rotary.  ``meta.positions`` is ``[T]`` (one rotary axis,
        fused kernel) or ``[3, T]`` (temporal / height / width axes of a vision-language prompt)."""
        c = self.cfg
        qkv = self._proj(h, "qkv_proj")
        if self.qkv_bias is not None:
            qkv = qkv + self.qkv_bias
        cached = meta.mode in ("decode", "prefill") and meta.k_cache is not None
        if cached and (meta.positions is None or meta.positions.dim() == 1):
            from unirl_b200.ops.rope import qk_norm_rope_cached

            # rotary + KV-cache write in one pass; decode keeps no dense k / v at all (attention reads the cache)
            return qk_norm_rope_cached(qkv, self.q_norm, self.k_norm, meta.positions, self.n_q, self.n_kv, c.head_dim, c.rope_theta, c.rms_norm_eps,
                                       meta.k_cache[self.layer_idx], meta.v_cache[self.layer_idx], meta.slot_mapping, dense_kv=meta.mode == "prefill")
        if meta.positions is not None and meta.positions.dim() == 2:
            from unirl_b200.ops.rope import mrope_qk

            q, k, v = mrope_qk(qkv, self.q_norm, self.k_norm, meta.positions, self.n_q, self.n_kv, c.head_dim, c.rope_theta, c.rms_norm_eps,
                               getattr(c, "mrope_section", (c.head_dim // 8, 3 * c.head_dim // 16, 3 * c.head_dim // 16)))
        else:
            q, k, v = qk_norm_rope(qkv, self.q_norm, self.k_norm, meta.positions, self.n_q, self.n_kv, c.head_dim, c.rope_theta, c.rms_norm_eps)
        if cached:
            A.kv_cache_write(k, v, meta.k_cache[self.layer_idx], meta.v_cache[self.layer_idx], meta.slot_mapping)
        return q, k, v

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: AttnMeta) -> torch.Tensor:
        """The KV cache (decode / prefill) has already been written by :meth:`_qkv_rope`."""
        if meta.mode == "decode" and meta.cascade is not None:
            return A.paged_decode_attention_cascade(q, meta.k_cache[self.layer_idx], meta.v_cache[self.layer_idx], meta.cascade, self.scale,
                                                    meta.workspace, meta.max_kv_len)
        if meta.mode == "decode":
            return A.paged_decode_attention(q, meta.k_cache[self.layer_idx], meta.v_cache[self.layer_idx], meta.block_tables,
                                            meta.seq_lens, self.scale, meta.workspace, meta.max_kv_len)
        if meta.cp_plan is not None:
            from unirl_b200.parallel.context_parallel import packed_attention

            return packed_attention(q, k, v, meta.cp_plan, meta.cp_comm, self.scale)
        return A.varlen_attention(q, k, v, meta.cu_seqlens, meta.max_seqlen, True, self.scale, meta.seq_lens_host)

    def forward_infer(self, pending: Optional[torch.Tensor], x: torch.Tensor, meta: AttnMeta) -> Tuple[torch.Tensor, torch.Tensor]:
        """Inference path on one GPU: the residual add of a projection output is deferred and fused with the NEXT RMSNorm
        (``add_rmsnorm``), so a block is 4 GEMMs + rope/cache + attention + 2 add-norms + SwiGLU.  ``pending`` is the previous
        block's un-added down-projection output; returns ``(pending', x')`` for the next block."""
        c = self.cfg
        if pending is None:
            h = rmsnorm(x, self.input_layernorm, c.rms_norm_eps)
        else:
            h, x = add_rmsnorm(pending, x, self.input_layernorm, c.rms_norm_eps)
        q, k, v = self._qkv_rope(h, meta)
        attn = self.attention(q, k, v, meta).reshape(x.shape[0], self.n_q * c.head_dim)
        h, x = add_rmsnorm(self._proj(attn, "o_proj"), x, self.post_attention_layernorm, c.rms_norm_eps)
        return self._proj(self._gate_up_act(h), "down_proj"), x

    def forward_fused_tp(self, x: torch.Tensor, h: torch.Tensor, meta: AttnMeta, next_norm: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Inference path under tensor parallelism: every row-parallel projection, its all-reduce, the residual add
        and the following RMSNorm run as one GEMM plus one peer-memory kernel.  ``h`` is the already normed input;
        returns the new residual stream and the input of the next block normed with ``next_norm``."""
        c, fused = self.cfg, self.tp.fused
        q, k, v = self._qkv_rope(h, meta)
        attn = self.attention(q, k, v, meta).reshape(x.shape[0], self.n_q * c.head_dim)
        x, h = fused.proj_reduce_norm(attn, self.o_proj, x, self.post_attention_layernorm, c.rms_norm_eps)
        return fused.proj_reduce_norm(self._gate_up_act(h), self.down_proj, x, next_norm, c.rms_norm_eps)

    def forward(self, x: torch.Tensor, meta: AttnMeta) -> torch.Tensor:
        c = self.cfg
        h = rmsnorm(x, self.input_layernorm, c.rms_norm_eps)
        q, k, v = self._qkv_rope(h, meta)
        attn = self.attention(q, k, v, meta).reshape(x.shape[0], self.n_q * c.head_dim)
        if self.tp.size == 1:
            x = self._proj(attn, "o_proj", residual=x)
        else:
            x = x + self.tp.reduce(self._proj(attn, "o_proj"))
        h = rmsnorm(x, self.post_attention_layernorm, c.rms_norm_eps)
        act = swiglu(self._proj(h, "gate_up_proj"))
        if self.tp.size == 1:
            return self._proj(act, "down_proj", residual=x)
        return x + self.tp.reduce(self._proj(act, "down_proj"))


class Qwen3Transformer(nn.Module):
    """Embedding → N decoder layers → final norm; ``lm_head`` kept as a parameter for the fused log-prob op."""

    block_class_name = "Qwen3DecoderLayer"
    _no_split_modules = ["Qwen3DecoderLayer"]

    def __init__(self, cfg: Qwen3Config, dtype: torch.dtype = torch.bfloat16, device: Any = "cpu", tp: Optional[TPContext] = None,
                 gradient_checkpointing: bool = False):
        super().__init__()
        self.cfg = cfg
        self.cp: Optional[Any] = None  # context-parallel group (parallel.context_parallel.ContextParallel) for the training replay; set by the trainer backend
        self.tp = tp or TPContext()
        self.gradient_checkpointing = gradient_checkpointing
        self.checkpoint_layers: Optional[int] = None  # recompute only the first N blocks in backward (None = all): 180 GB of HBM holds the rest
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        self.layers = nn.ModuleList(Qwen3DecoderLayer(cfg, i, self.tp, dtype, device) for i in range(cfg.num_hidden_layers))
        self.norm = nn.Parameter(torch.empty(cfg.hidden_size, dtype=dtype, device=device))
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        if cfg.tie_word_embeddings:
            self.embed_tokens._wgrad_shared = True  # gradient arrives from the embedding lookup AND the output projection

    # ---- init ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "Qwen3Transformer":
        """Deterministic random init, generated on the parameter's device (normal(0, std); norms = 1).

        The stream depends only on ``(seed, parameter name)`` so TP shards of different ranks and the
        unsharded trainer copy do NOT coincide — use :func:`shard_from_full` for consistent shards.
        """
        for i, (name, p) in enumerate(self.named_parameters()):
            if p.dim() == 1:
                p.zero_() if name.endswith("bias") else p.fill_(1.0)
            else:
                g = torch.Generator(device=p.device)
                g.manual_seed(seed * 100003 + i)
                p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=g))
        return self

    @property
    def output_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    # ---- forward -------------------------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, meta: AttnMeta) -> torch.Tensor:
        """``tokens [T]`` → final-normed hidden states ``[T, H]``."""
        x = self.embed_tokens[tokens] if meta.input_embeds is None else meta.input_embeds.to(self.embed_tokens.dtype)
        if self.tp.size > 1 and self.tp.fused is not None and not torch.is_grad_enabled() and x.is_cuda \
                and not any(getattr(l, "_lora_index", None) for l in self.layers):
            h = rmsnorm(x, self.layers[0].input_layernorm, self.cfg.rms_norm_eps)
            for i, layer in enumerate(self.layers):
                nxt = self.layers[i + 1].input_layernorm if i + 1 < len(self.layers) else self.norm
                x, h = layer.forward_fused_tp(x, h, meta, nxt)
            return h
        if not torch.is_grad_enabled() and x.is_cuda and self.tp.size == 1 and meta.mode in ("decode", "prefill"):
            pending = None
            for layer in self.layers:
                pending, x = layer.forward_infer(pending, x, meta)
            h, _ = add_rmsnorm(pending, x, self.norm, self.cfg.rms_norm_eps)
            return h
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled() and meta.mode == "train"
        n_ckpt = len(self.layers) if self.checkpoint_layers is None else int(self.checkpoint_layers)
        for i, layer in enumerate(self.layers):
            if ckpt and i < n_ckpt:
                x = torch.utils.checkpoint.checkpoint(layer, x, meta, use_reentrant=False)
            else:
                x = layer(x, meta)
        return rmsnorm(x, self.norm, self.cfg.rms_norm_eps)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return linear(hidden, self.output_weight)

    # ---- Hugging Face key grammar ---------------------------------------------------------------------
    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        """Un-fuse into HF names (TP shards export their local slices)."""
        c, out = self.cfg, {}
        out["model.embed_tokens.weight"] = self.embed_tokens
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            q, k, v = l.qkv_proj.split([l.n_q * c.head_dim, l.n_kv * c.head_dim, l.n_kv * c.head_dim], 0)
            g, u = l.gate_up_proj.split([l.inter, l.inter], 0)
            out.update({p + "input_layernorm.weight": l.input_layernorm, p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k,
                        p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": l.o_proj,
                        p + "post_attention_layernorm.weight": l.post_attention_layernorm, p + "mlp.gate_proj.weight": g,
                        p + "mlp.up_proj.weight": u, p + "mlp.down_proj.weight": l.down_proj})
            if l.q_norm is not None:
                out[p + "self_attn.q_norm.weight"], out[p + "self_attn.k_norm.weight"] = l.q_norm, l.k_norm
            if l.qkv_bias is not None:
                nq, nkv = l.n_q * c.head_dim, l.n_kv * c.head_dim
                out[p + "self_attn.q_proj.bias"], out[p + "self_attn.k_proj.bias"], out[p + "self_attn.v_proj.bias"] = l.qkv_bias.split([nq, nkv, nkv])
        out["model.norm.weight"] = self.norm
        if self.lm_head is not None:
            out["lm_head.weight"] = self.lm_head
        return out

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> None:
        """Load full (unsharded) HF tensors, slicing out this rank's TP shard."""
        c, tp = self.cfg, self.tp
        rows = lambda w, n: w.view(tp.size, n, *w.shape[1:])[tp.rank] if tp.size > 1 else w  # noqa: E731
        cols = lambda w, n: w.view(w.shape[0], tp.size, n)[:, tp.rank] if tp.size > 1 else w  # noqa: E731
        self.embed_tokens.copy_(sd["model.embed_tokens.weight"])
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            l.input_layernorm.copy_(sd[p + "input_layernorm.weight"])
            l.post_attention_layernorm.copy_(sd[p + "post_attention_layernorm.weight"])
            l.qkv_proj.copy_(torch.cat([rows(sd[p + "self_attn.q_proj.weight"], l.n_q * c.head_dim),
                                        rows(sd[p + "self_attn.k_proj.weight"], l.n_kv * c.head_dim),
                                        rows(sd[p + "self_attn.v_proj.weight"], l.n_kv * c.head_dim)], 0))
            l.o_proj.copy_(cols(sd[p + "self_attn.o_proj.weight"], l.n_q * c.head_dim))
            l.gate_up_proj.copy_(torch.cat([rows(sd[p + "mlp.gate_proj.weight"], l.inter), rows(sd[p + "mlp.up_proj.weight"], l.inter)], 0))
            l.down_proj.copy_(cols(sd[p + "mlp.down_proj.weight"], l.inter))
            if l.q_norm is not None:
                l.q_norm.copy_(sd[p + "self_attn.q_norm.weight"])
                l.k_norm.copy_(sd[p + "self_attn.k_norm.weight"])
            if l.qkv_bias is not None:
                l.qkv_bias.copy_(torch.cat([rows(sd[p + "self_attn.q_proj.bias"], l.n_q * c.head_dim), rows(sd[p + "self_attn.k_proj.bias"], l.n_kv * c.head_dim),
                                            rows(sd[p + "self_attn.v_proj.bias"], l.n_kv * c.head_dim)], 0))
        self.norm.copy_(sd["model.norm.weight"])
        if self.lm_head is not None:
            self.lm_head.copy_(sd.get("lm_head.weight", sd["model.embed_tokens.weight"]))


def tp_slice_spec(name: str, cfg: Qwen3Config) -> Tuple[str, Tuple[int, ...]]:
    """How a *fused native* parameter shards under TP: ``("rows", sections)`` | ``("cols", ())`` | ``("replicate", ())``.

    ``sections`` are the row-block sizes of the fused weight that must each be split (q|k|v, gate|up).
    """
    d = cfg.head_dim
    leaf = name.rsplit(".", 1)[-1]
    if name.startswith("visual.") or ".visual." in name:  # the vision tower of a vision-language model is whole on every rank
        return "replicate", ()
    if leaf in ("qkv_proj", "qkv_bias"):
        return "rows", (cfg.num_attention_heads * d, cfg.num_key_value_heads * d, cfg.num_key_value_heads * d)
    if leaf == "gate_up_proj":
        return "rows", (cfg.intermediate_size, cfg.intermediate_size)
    if leaf in ("o_proj", "down_proj"):
        return "cols", ()
    return "replicate", ()


@torch.no_grad()
def shard_param(full: torch.Tensor, name: str, cfg: Qwen3Config, tp_rank: int, tp_size: int) -> torch.Tensor:
    """This rank's TP shard of a full fused parameter (view/cat of views; reference for the reshard kernel)."""
    kind, sections = tp_slice_spec(name, cfg)
    if tp_size == 1 or kind == "replicate":
        return full
    if kind == "cols":
        n = full.shape[1] // tp_size
        return full[:, tp_rank * n : (tp_rank + 1) * n]
    parts, row = [], 0
    for s in sections:
        n = s // tp_size
        parts.append(full[row + tp_rank * n : row + (tp_rank + 1) * n])
        row += s
    return torch.cat(parts, 0)


__all__ = ["Qwen3Config", "Qwen3Transformer", "Qwen3DecoderLayer", "AttnMeta", "TPContext", "tp_slice_spec", "shard_param"]
