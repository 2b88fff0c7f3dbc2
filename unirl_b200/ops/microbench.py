"""Operator microbenchmarks with roofline fractions: ``python -m unirl_b200.ops.microbench <case> [options]``.

Cases
-----
``gemm``              bf16 ``A[M,K]·W[N,K]ᵀ`` — the tcgen05 kernel against the library GEMM of the same shape
``decode_attention``  paged-KV decode attention (memory-bound: bytes = K and V of every live token)
``linear_logprob``    fused ``lm_head → log-softmax → gather`` against materialised logits
``linear_sample``     fused ``lm_head → Gumbel-max sampling``
``elementwise``       RMSNorm / QK-norm+RoPE / SwiGLU streaming kernels
``decode_step``       one whole decode step of the Qwen3-4B-shaped policy at a fixed context (eager and CUDA-graph replay)
``attention``         causal self-attention forward / backward over packed sequences vs the dense library kernels
``train_step``        forward + backward of one training micro-batch of the Qwen3-4B-shaped policy
``peer``              (under ``torchrun``) fused peer-memory collectives against their NCCL compositions

Timing: CUDA events on the launching stream, ≥3 warm-up iterations, a 256 MiB buffer is rewritten between timed
iterations to flush L2 (the L2 is 126 MB), best and median of ``--iters`` are reported, max over ranks for ``peer``.
Peaks come from ``MEASURED_PEAKS.json`` at the repository root when present (fractions are "of measured"),
otherwise 6.65 TB/s and 1.59 PFLOP/s ("of fallback").  One JSON line per result on stdout.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
from typing import Any, Callable, Dict, List

import torch


def _peaks() -> Dict[str, Any]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]), "kind": "of measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "kind": "of fallback"}


class _Timer:
    def __init__(self, iters: int, flush: bool = True):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn: Callable[[], Any], warmup: int = 3) -> Dict[str, float]:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts: List[float] = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return {"best_ms": min(ts), "median_ms": statistics.median(ts)}


def _emit(row: Dict[str, Any]) -> None:
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)


# ---------------------------------------------------------------------------------------------------------- cases
def case_gemm(args: argparse.Namespace) -> None:
    from unirl_b200.ops._ext import require_ext

    C, pk, timer = require_ext(), _peaks(), _Timer(args.iters)
    shapes = [tuple(int(x) for x in s.split("x")) for s in args.shapes.split(",")]
    for m, n, k in shapes:
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * m * n * k
        ours = timer(lambda: C.gemm_bf16_tn(a, w, None, 0))
        row = {"case": "gemm", "M": m, "N": n, "K": k, "tcgen05_ms": ours["best_ms"], "tcgen05_tflops": fl / ours["best_ms"] / 1e9,
               "frac_of_peak": fl / ours["best_ms"] / 1e9 / pk["tflops"], "peak": pk["kind"]}
        if not args.no_library:
            lib = timer(lambda: torch.nn.functional.linear(a, w))
            row.update(library_ms=lib["best_ms"], library_tflops=fl / lib["best_ms"] / 1e9)
        assert C.gemm_status(True) == 0, "a pipeline wait timed out"
        _emit(row)


def case_gemm_bwd(args: argparse.Namespace) -> None:
    """The two backward GEMMs of ``Y[M,N] = X[M,K]·W[N,K]ᵀ`` for every forward shape given: ``dX = dY·W`` (W read as stored) and
    ``dW += dYᵀ·X`` (both read as stored, fp32 accumulation in the epilogue) on the tcgen05 kernel vs the library calls."""
    from unirl_b200.ops._ext import require_ext

    C, pk, timer = require_ext(), _peaks(), _Timer(args.iters)
    shapes = [tuple(int(x) for x in s.split("x")) for s in args.shapes.split(",")]
    for m, n, k in shapes:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        gy = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
        acc = torch.zeros(n, k, device="cuda", dtype=torch.float32)
        fl = 2.0 * m * n * k
        dx = timer(lambda: C.gemm_bf16(gy, w, False, True))
        dw = timer(lambda: C.gemm_bf16(gy, x, True, True, acc, True))
        row = {"case": "gemm_bwd", "M": m, "N": n, "K": k, "dx_ms": dx["best_ms"], "dx_tflops": fl / dx["best_ms"] / 1e9, "dw_ms": dw["best_ms"],
               "dw_tflops": fl / dw["best_ms"] / 1e9, "peak": pk["kind"], "peak_tflops": pk["tflops"]}
        if not args.no_library:
            ldx = timer(lambda: gy @ w)
            ldw = timer(lambda: torch.addmm(acc, gy.t(), x, out_dtype=torch.float32, out=acc))
            row.update(library_dx_tflops=fl / ldx["best_ms"] / 1e9, library_dw_tflops=fl / ldw["best_ms"] / 1e9)
        assert C.gemm_status(True) == 0, "a pipeline wait timed out"
        _emit(row)


def case_skinny_gemm(args: argparse.Namespace) -> None:
    """Decode-shaped GEMMs (weight-bandwidth bound): cluster split-K tcgen05 kernel vs the library GEMM, each timed over a ring of
    distinct weight matrices larger than L2 so every call streams its weights from HBM."""
    from unirl_b200.ops._ext import require_ext

    C, pk = require_ext(), _peaks()
    timer = _Timer(args.iters, flush=False)
    shapes = [tuple(int(x) for x in s.split("x")) for s in (args.skinny_shapes or "128x6144x2560,128x2560x4096,128x19456x2560,128x2560x9728,256x2560x9728").split(",")]
    for m, n, k in shapes:
        ring = max(2, int(400e6 // (n * k * 2)) + 1)
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        ws = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05 for _ in range(ring)]
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

        def ours():
            for w in ws:
                C.gemm_bf16_tn_skinny(a, w, None, out)

        def lib():
            for w in ws:
                torch.matmul(a, w.t(), out=out)

        t_ours, t_lib = timer(ours), timer(lib)
        gb = (n * k + m * k + m * n) * 2 / 1e9
        assert C.gemm_status(True) == 0, "a pipeline wait timed out"
        _emit({"case": "skinny_gemm", "M": m, "N": n, "K": k, "tile_n": C.gemm_skinny_plan(m, n, k, False)[0], "cluster": C.gemm_skinny_plan(m, n, k, False)[1], "skinny_us": t_ours["best_ms"] / ring * 1e3,
               "library_us": t_lib["best_ms"] / ring * 1e3, "skinny_gbs": gb / (t_ours["best_ms"] / ring) * 1e3,
               "frac_of_peak": gb / (t_ours["best_ms"] / ring) * 1e3 / pk["hbm_gbs"], "library_gbs": gb / (t_lib["best_ms"] / ring) * 1e3, "peak": pk["kind"]})


def case_decode_attention(args: argparse.Namespace) -> None:
    from unirl_b200.ops.attention import paged_decode_attention

    pk, timer = _peaks(), _Timer(args.iters)
    b, ctx, hq, hkv, d, ps = args.batch, args.ctx, args.q_heads, args.kv_heads, args.head_dim, args.page_size
    pages_per = (ctx + ps - 1) // ps
    n_pages = b * pages_per
    kc = torch.randn(n_pages, hkv, ps, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(n_pages, device="cuda").view(b, pages_per).to(torch.int32)
    sl = torch.full((b,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(b, hq, d, device="cuda", dtype=torch.bfloat16)
    ws = torch.empty(b * hq * 32 * (d + 2), device="cuda")
    t = timer(lambda: paged_decode_attention(q, kc, vc, bt, sl, None, ws, ctx))
    gb = 2.0 * b * ctx * hkv * d * 2 / 1e9
    _emit({"case": "decode_attention", "batch": b, "ctx": ctx, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "page_size": ps, "kv_gb": gb,
           "best_ms": t["best_ms"], "median_ms": t["median_ms"], "gbs": gb / t["best_ms"] * 1e3, "frac_of_peak": gb / t["best_ms"] * 1e3 / pk["hbm_gbs"],
           "peak": pk["kind"]})


def case_linear_logprob(args: argparse.Namespace) -> None:
    from unirl_b200.ops.logprob import linear_logprob

    pk, timer = _peaks(), _Timer(args.iters)
    t_, h, v = args.tokens, args.hidden, args.vocab
    x = torch.randn(t_, h, device="cuda", dtype=torch.bfloat16) * 0.5
    w = torch.randn(v, h, device="cuda", dtype=torch.bfloat16) * 0.02
    tgt = torch.randint(0, v, (t_,), device="cuda")
    fused = timer(lambda: linear_logprob(x, w, tgt, 1.0))

    def unfused():
        z = torch.nn.functional.linear(x, w).float()
        return torch.log_softmax(z, -1).gather(-1, tgt[:, None])

    lib = timer(unfused)
    fl = 2.0 * t_ * h * v
    _emit({"case": "linear_logprob", "tokens": t_, "hidden": h, "vocab": v, "fused_ms": fused["best_ms"], "fused_tflops": fl / fused["best_ms"] / 1e9,
           "frac_of_peak": fl / fused["best_ms"] / 1e9 / pk["tflops"], "peak": pk["kind"], "materialised_logits_ms": lib["best_ms"],
           "logits_bytes_avoided_gb": t_ * v * (2 + 4 + 4) / 1e9})


def case_linear_sample(args: argparse.Namespace) -> None:
    from unirl_b200.ops.sampling import linear_sample

    pk, timer = _peaks(), _Timer(args.iters)
    b, h, v = args.batch, args.hidden, args.vocab
    x = torch.randn(b, h, device="cuda", dtype=torch.bfloat16) * 0.5
    w = torch.randn(v, h, device="cuda", dtype=torch.bfloat16) * 0.02
    t = timer(lambda: linear_sample(x, w, 1.0, 0, 1.0, seed=1, step=3))
    gb = v * h * 2 / 1e9
    _emit({"case": "linear_sample", "batch": b, "hidden": h, "vocab": v, "best_ms": t["best_ms"], "weight_gbs": gb / t["best_ms"] * 1e3,
           "frac_of_peak": gb / t["best_ms"] * 1e3 / pk["hbm_gbs"], "peak": pk["kind"]})


def require_ext_():
    from unirl_b200.ops._ext import require_ext

    return require_ext()


def case_elementwise(args: argparse.Namespace) -> None:
    from unirl_b200.ops.activation import swiglu
    from unirl_b200.ops.norm import rmsnorm
    from unirl_b200.ops.rope import qk_norm_rope

    pk, timer = _peaks(), _Timer(args.iters)
    t_, h = args.tokens, args.hidden
    x = torch.randn(t_, h, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    r = timer(lambda: rmsnorm(x, w, 1e-6))
    _emit({"case": "rmsnorm", "tokens": t_, "hidden": h, "best_ms": r["best_ms"], "gbs": 2 * x.numel() * 2 / r["best_ms"] / 1e6,
           "frac_of_peak": 2 * x.numel() * 2 / r["best_ms"] / 1e6 / pk["hbm_gbs"], "peak": pk["kind"]})
    C = require_ext_()
    gy, rstd = torch.randn_like(x), torch.rand(t_, device="cuda") + 0.5
    r = timer(lambda: C.rmsnorm_bwd(gy, x, w, rstd))
    _emit({"case": "rmsnorm_bwd", "tokens": t_, "hidden": h, "best_ms": r["best_ms"], "gbs": 3 * x.numel() * 2 / r["best_ms"] / 1e6,
           "frac_of_peak": 3 * x.numel() * 2 / r["best_ms"] / 1e6 / pk["hbm_gbs"], "peak": pk["kind"]})
    inter = args.intermediate
    gu = torch.randn(t_, 2 * inter, device="cuda", dtype=torch.bfloat16)
    r = timer(lambda: swiglu(gu))
    _emit({"case": "swiglu", "tokens": t_, "intermediate": inter, "best_ms": r["best_ms"], "gbs": 3 * t_ * inter * 2 / r["best_ms"] / 1e6,
           "frac_of_peak": 3 * t_ * inter * 2 / r["best_ms"] / 1e6 / pk["hbm_gbs"], "peak": pk["kind"]})
    hq, hkv, d = args.q_heads, args.kv_heads, args.head_dim
    qkv = torch.randn(t_, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
    qw, kw = torch.ones(d, device="cuda", dtype=torch.bfloat16), torch.ones(d, device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(t_, device="cuda") % 4096
    r = timer(lambda: qk_norm_rope(qkv, qw, kw, pos, hq, hkv, d, 1e6, 1e-6))
    _emit({"case": "qk_norm_rope", "tokens": t_, "best_ms": r["best_ms"], "gbs": 2 * qkv.numel() * 2 / r["best_ms"] / 1e6,
           "frac_of_peak": 2 * qkv.numel() * 2 / r["best_ms"] / 1e6 / pk["hbm_gbs"], "peak": pk["kind"]})


def case_decode_step(args: argparse.Namespace) -> None:
    """One full decode step of the Qwen3-4B-shaped policy (36 blocks + fused lm_head sampling) at a fixed context length, eager launches
    (so a profiler can list kernels) and replayed from a CUDA graph (what the rollout engine runs)."""
    from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer
    from unirl_b200.ops._ext import require_ext
    from unirl_b200.ops.sampling import linear_sample
    from unirl_b200.rollout.engine.native_ar.kv_cache import PagedKVCache

    pk = _peaks()
    cfg = Qwen3Config.qwen3_4b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    b, ctx, ps = args.batch, args.ctx, args.page_size
    tp, tpc, far = int(os.environ.get("WORLD_SIZE", "1")), None, None
    if tp > 1:  # under torchrun: the ranks form one tensor-parallel group with the fused all-reduce of the rollout engine
        import torch.distributed as dist

        from unirl_b200.distributed.group.comm import Comm
        from unirl_b200.models.qwen3.modeling import TPContext
        from unirl_b200.parallel.fused_collectives import FusedAllReduce

        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
        far = FusedAllReduce(Comm.world(), max(b, 64), cfg.hidden_size, torch.device("cuda", local))
        tpc = TPContext(int(os.environ["RANK"]), tp, far, fused=far)
    model = Qwen3Transformer(cfg, dtype=torch.bfloat16, device="cuda", tp=tpc).init_weights(0).eval().requires_grad_(False)
    pages_per = (ctx + 1 + ps - 1) // ps
    cache = PagedKVCache(cfg.num_hidden_layers, cfg.num_key_value_heads // tp, cfg.head_dim, ps, b * pages_per, torch.bfloat16, "cuda")
    for t in cache.k + cache.v:
        t.normal_()
    bt = torch.randperm(b * pages_per, device="cuda").view(b, pages_per).to(torch.int32)
    pos = torch.full((b,), ctx, dtype=torch.long, device="cuda")
    page = bt.gather(1, (pos // ps).unsqueeze(1)).squeeze(1).long()
    meta = AttnMeta(mode="decode", positions=pos, k_cache=cache.k, v_cache=cache.v, block_tables=bt, seq_lens=(pos + 1).to(torch.int32),
                    slot_mapping=page * ps + pos % ps, max_kv_len=ctx + 1)
    C = require_ext()
    meta.workspace = torch.empty(C.decode_workspace_size(b, cfg.num_attention_heads // tp, cfg.head_dim, ctx + 1), dtype=torch.float32, device="cuda")
    tokens = torch.randint(0, cfg.vocab_size, (b,), device="cuda")

    @torch.no_grad()
    def step():
        h = model(tokens, meta)
        return linear_sample(h, model.output_weight, 1.0, 0, 1.0, seed=1, step=3)

    eager = _Timer(args.iters, flush=False)(step)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    if far is not None:
        far.align()
    with torch.cuda.graph(g, stream=s):
        step()
        if far is not None:
            far.align()
    graphed = _Timer(args.iters, flush=False)(g.replay)
    if far is not None:
        far.arena.check()
    n_param = sum(p.numel() for n, p in model.named_parameters() if not n.startswith("embed_tokens"))
    gb = (n_param * 2 + 2.0 * b * ctx * (cfg.num_key_value_heads // tp) * cfg.head_dim * 2 * cfg.num_hidden_layers) / 1e9
    if int(os.environ.get("RANK", "0")) == 0:
        _emit({"case": "decode_step", "tp": tp, "batch": b, "ctx": ctx, "layers": cfg.num_hidden_layers, "eager_ms": eager["median_ms"],
               "graph_ms": graphed["median_ms"], "weights_plus_kv_gb_per_gpu": gb, "gbs": gb / graphed["median_ms"] * 1e3,
               "frac_of_peak": gb / graphed["median_ms"] * 1e3 / pk["hbm_gbs"], "peak": pk["kind"]})
    if tp > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def case_train_step(args: argparse.Namespace) -> None:
    """Forward + backward of one training micro-batch of the Qwen3-4B-shaped policy (packed sequences, fused lm_head log-prob), no recompute."""
    from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer
    from unirl_b200.ops.logprob import linear_logprob

    pk = _peaks()
    cfg = Qwen3Config.qwen3_4b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    nseq, l = args.seqs, args.ctx
    model = Qwen3Transformer(cfg, dtype=torch.bfloat16, device="cuda").init_weights(0)
    tokens = torch.randint(0, cfg.vocab_size, (nseq * l,), device="cuda")
    pos = torch.arange(l, device="cuda").repeat(nseq)
    cu = torch.arange(0, (nseq + 1) * l, l, device="cuda", dtype=torch.int32)
    idx = torch.arange(600, nseq * l - 1, device="cuda")

    def step():
        h = model(tokens, AttnMeta(mode="train", positions=pos, cu_seqlens=cu, max_seqlen=l, seq_lens_host=[l] * nseq))
        linear_logprob(h.index_select(0, idx), model.output_weight, tokens[idx + 1], 1.0).mean().backward()
        for p_ in model.parameters():
            p_.grad = None

    t = _Timer(args.iters, flush=False)(step, warmup=2)
    ntok = nseq * l
    dense = cfg.num_params() - 2 * cfg.vocab_size * cfg.hidden_size
    flops = 6.0 * ntok * dense + 6.0 * idx.numel() * cfg.vocab_size * cfg.hidden_size + 3.0 * 4 * l * l / 2 * cfg.head_dim * cfg.num_attention_heads * cfg.num_hidden_layers * nseq
    _emit({"case": "train_step", "seqs": nseq, "seq_len": l, "layers": cfg.num_hidden_layers, "median_ms": t["median_ms"], "tokens_per_s": ntok / t["median_ms"] * 1e3,
           "model_tflops": flops / t["median_ms"] / 1e9, "frac_of_peak": flops / t["median_ms"] / 1e9 / pk["tflops"], "peak": pk["kind"]})


def case_attention(args: argparse.Namespace) -> None:
    """Causal self-attention forward + backward over a micro-batch of equal-length sequences: the packed-sequence op against the
    dense library kernel on the same (padded) problem."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from unirl_b200.ops.attention import varlen_attention

    pk = _peaks()
    b, l, hq, hkv, d = args.seqs, args.ctx, args.q_heads, args.kv_heads, args.head_dim
    q = torch.randn(b * l, hq, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b * l, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b * l, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.arange(0, (b + 1) * l, l, device="cuda", dtype=torch.int32)
    go = torch.randn(b * l, hq, d, device="cuda", dtype=torch.bfloat16)
    flops_f = 4.0 * l * l / 2 * d * hq * b
    timer = _Timer(args.iters, flush=False)
    lens = [l] * b if not args.ragged else None  # --ragged: dispatch without host lengths (packed kernel)

    def packed():
        varlen_attention(q, k, v, cu, l, True, None, lens).backward(go)
        q.grad = k.grad = v.grad = None

    def packed_fwd():
        with torch.no_grad():
            varlen_attention(q, k, v, cu, l, True, None, lens)

    row = {"case": "attention", "seqs": b, "seq_len": l, "q_heads": hq, "kv_heads": hkv, "head_dim": d}
    t = timer(packed_fwd)
    row.update(packed_fwd_ms=t["median_ms"], packed_fwd_tflops=flops_f / t["median_ms"] / 1e9)
    t = timer(packed)
    row.update(packed_fwd_bwd_ms=t["median_ms"], packed_fwd_bwd_tflops=3.5 * flops_f / t["median_ms"] / 1e9)
    qd, kd, vd = (x.detach().view(b, l, -1, d).transpose(1, 2).contiguous().requires_grad_() for x in (q, k, v))
    god = go.view(b, l, hq, d).transpose(1, 2).contiguous()
    for name, backend in (("cudnn", SDPBackend.CUDNN_ATTENTION), ("flash", SDPBackend.FLASH_ATTENTION)):
        try:
            def dense():
                with sdpa_kernel(backend):
                    F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=hq != hkv).backward(god)
                qd.grad = kd.grad = vd.grad = None

            t = timer(dense)
            row.update({f"dense_{name}_fwd_bwd_ms": t["median_ms"], f"dense_{name}_fwd_bwd_tflops": 3.5 * flops_f / t["median_ms"] / 1e9})
        except Exception as e:  # noqa: BLE001
            row[f"dense_{name}_error"] = str(e)[:120]
    try:
        def dense_fwd():
            with torch.no_grad(), sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=hq != hkv)

        t = timer(dense_fwd)
        row.update(dense_cudnn_fwd_ms=t["median_ms"], dense_cudnn_fwd_tflops=flops_f / t["median_ms"] / 1e9)
    except Exception as e:  # noqa: BLE001
        row["dense_cudnn_fwd_error"] = str(e)[:120]
    row.update(frac_of_peak=row["packed_fwd_bwd_tflops"] / pk["tflops"], peak=pk["kind"])
    from unirl_b200.ops._ext import require_ext

    C = require_ext()
    if C.attn_diag(False, True):  # a build with phase timers (-DUNIRL_B200_ATTN_DIAG): one clean forward + backward, cycles per phase summed over CTAs
        C.attn_diag(True, True)
        packed()
        torch.cuda.synchronize()
        f, bw = C.attn_diag(False, True), C.attn_diag(True, True)
        row["diag_fwd_issuer"] = dict(zip(("start", "wait_v", "wait_p0", "wait_p1", "wait_k", "issue"), f[32:38]))
        for t in (0, 1):
            row[f"diag_fwd_softmax{t}"] = dict(zip(("wait_s", "pass1_max", "rescale", "pass2_exp", "st_arrive", "wait_o", "epilogue"), f[40 + 8 * t : 47 + 8 * t]))
        row["diag_bwd_issuer"] = dict(zip(("start", "wait_p", "wait_qdo", "wait_ds", "wait_free"), bw[0:5]))
        row["diag_bwd_compute"] = dict(zip(("stats", "wait_s", "phase_a", "wait_dp", "phase_b"), bw[8:13]))
        row["diag_bwd_drain"] = dict(zip(("wait_dq", "dq_read", "dq_stage", "wait_reads"), bw[16:20]))
    _emit(row)


def case_peer(args: argparse.Namespace) -> None:
    """Fused peer-memory collectives vs their NCCL compositions (run under torchrun, one rank per GPU)."""
    import torch.distributed as dist

    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.ops.norm import rmsnorm
    from unirl_b200.parallel.fused_collectives import FusedAllReduce, PeerArena
    from unirl_b200.ops._ext import require_ext

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
    comm, dev, C = Comm.world(), torch.device("cuda", local), require_ext()
    timer = _Timer(args.iters, flush=False)

    def tmax(x: float) -> float:
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # -- TP decode: row-parallel projection + all-reduce + residual + RMSNorm
    T, H, K = args.batch, args.hidden, args.hidden // world
    inp = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(H, K, device=dev, dtype=torch.bfloat16) * 0.02
    res = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    far = FusedAllReduce(comm, max(T, 64), H, dev)

    def fused_pair():
        far.proj_reduce_norm(inp, w, res, nw, 1e-6)
        far.proj_reduce_norm(inp, w, res, nw, 1e-6)

    def nccl_pair():
        for _ in range(2):
            y = torch.matmul(inp, w.t())
            dist.all_reduce(y)
            x = y + res
            rmsnorm(x, nw, 1e-6)

    f, n = timer(fused_pair), timer(nccl_pair)
    far.arena.check()
    fb, nb = tmax(f["median_ms"]) / 2, tmax(n["median_ms"]) / 2
    if rank == 0:
        _emit({"case": "peer_tp_proj_allreduce_add_norm", "world": world, "tokens": T, "hidden": H, "fused_us": fb * 1e3, "nccl_composition_us": nb * 1e3,
               "speedup": nb / fb})
    # -- trainer: reduce-scatter (+mean +sum of squares) and AdamW + publish over a group of `numel` parameters
    numel = args.numel // (world * 128) * (world * 128)
    shard = numel // world
    ga = PeerArena(comm, numel * 4 + 4096, dev, wait_s=20.0)
    pa = PeerArena(comm, numel * 2 + 4096, dev, wait_s=20.0)
    grad, replica = ga.take(numel, torch.float32), pa.take(numel, torch.bfloat16)
    grad.normal_()
    out, ss = torch.empty(shard, device=dev), torch.zeros(1, device=dev)
    master, m, v = torch.randn(shard, device=dev), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    clip = torch.ones(1, device=dev)
    dist.barrier()

    def fused_rs():
        C.peer_reduce_scatter_sumsq(ga.peer, grad, out, ss, 1.0 / world)

    def nccl_rs():
        dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.AVG)
        C.sum_squares(out)

    def fused_opt():
        C.peer_adamw_publish(pa.peer, replica, master, out, m, v, None, 1e-5, 0.9, 0.95, 1e-8, 0.0, 3, clip, 0.0)

    low = torch.empty(shard, device=dev, dtype=torch.bfloat16)

    def nccl_opt():
        C.adamw_step(master, out, m, v, low, None, 1e-5, 0.9, 0.95, 1e-8, 0.0, 3, 1.0, 0.0, clip)
        dist.all_gather_into_tensor(replica, low)

    rows = {}
    for name, fn in (("fused_reduce_scatter_norm", fused_rs), ("nccl_reduce_scatter_plus_norm", nccl_rs), ("fused_adamw_publish", fused_opt),
                     ("nccl_adamw_plus_all_gather", nccl_opt)):
        rows[name] = tmax(timer(fn)["median_ms"])
    ga.check()
    pa.check()
    if rank == 0:
        rs_bytes = (world - 1) * shard * 4  # bytes this rank pulls over NVLink
        ag_bytes = (world - 1) * shard * 2  # bytes this rank pushes over NVLink
        _emit({"case": "peer_trainer_collectives", "world": world, "numel": numel, **{k + "_ms": v for k, v in rows.items()},
               "rs_nvlink_gbs": rs_bytes / rows["fused_reduce_scatter_norm"] / 1e6, "publish_nvlink_gbs": ag_bytes / rows["fused_adamw_publish"] / 1e6,
               "nvlink_peer_copy_gbs_measured_reference": 770.0})
    # -- Ulysses exchange (sequence shard -> head shard) of one WAN-sized activation: 40 heads x 128, 32760 / 8 tokens per rank
    from unirl_b200.parallel.fused_collectives import FusedUlyssesExchange
    from unirl_b200.parallel.ulysses import _a2a_seq_to_head

    heads = 40 // world * world
    xa = torch.randn(1, 4095, heads, 128, device=dev, dtype=torch.bfloat16)
    ex = FusedUlyssesExchange(comm, dev, wait_s=20.0)
    f = tmax(timer(lambda: ex.exchange(xa, 0))["median_ms"])
    n = tmax(timer(lambda: _a2a_seq_to_head(xa, comm))["median_ms"])
    ex.check()
    if rank == 0:
        moved = xa.numel() * 2 * (world - 1) / world  # bytes this rank pulls over NVLink
        _emit({"case": "peer_ulysses_exchange", "world": world, "shape": list(xa.shape), "fused_ms": f, "library_pack_all_to_all_unpack_ms": n, "speedup": n / f,
               "nvlink_gbs": moved / f / 1e6, "nvlink_peer_copy_gbs_measured_reference": 770.0})
    # -- the same exchange inside the QKV projection: WAN-14B geometry (hidden 5120, 40 heads x 128, 32760 / 8 tokens per rank) and SD3.5-M
    # (hidden 1536, 24 heads x 64, 4096 / world tokens, batch 8); "separate" = projection GEMM, bias add, then the exchange kernel per q / k / v
    from unirl_b200.ops.linear import linear
    from unirl_b200.parallel.fused_collectives import FusedHeadScatterProjection

    sc = FusedHeadScatterProjection(comm, dev, wait_s=20.0)
    for label, (bsz, l, hidden, nh, hd) in (("wan14b", (1, 4095, 5120, 40 // world * world, 128)), ("sd35m", (8, 4096 // world, 1536, 24 // world * world, 64))):
        xin = torch.randn(bsz, l, hidden, device=dev, dtype=torch.bfloat16)
        wq = torch.randn(3 * nh * hd, hidden, device=dev, dtype=torch.bfloat16) * 0.02
        bq = torch.randn(3 * nh * hd, device=dev, dtype=torch.bfloat16)

        def separate():
            y = (linear(xin, wq) + bq).view(bsz, l, 3, nh, hd)
            return [ex.exchange(y[:, :, i].contiguous(), 0) for i in range(3)]

        def fused():
            return sc.project(xin, wq, bq, nh, hd, 3)

        def gemm_only():
            return linear(xin, wq)

        f, n, g = tmax(timer(fused)["median_ms"]), tmax(timer(separate)["median_ms"]), tmax(timer(gemm_only)["median_ms"])
        sc.check()
        ex.check()
        if rank == 0:
            moved = bsz * l * 3 * nh * hd * 2 * (world - 1) / world  # bytes this rank stores into its peers
            flops = 2.0 * bsz * l * hidden * 3 * nh * hd
            _emit({"case": "peer_qkv_projection_with_exchange", "geometry": label, "world": world, "tokens_per_rank": bsz * l, "fused_ms": f, "separate_ms": n, "gemm_alone_ms": g,
                   "speedup": n / f, "exchange_cost_over_gemm_ms": f - g, "fused_tflops": flops / f / 1e9, "nvlink_gbs_if_not_overlapped": moved / max(f - g, 1e-6) / 1e6,
                   "roofline_ms": max(flops / (_peaks()["tflops"] * 1e9), moved / 770e6), "nvlink_peer_copy_gbs_measured_reference": 770.0})
    dist.barrier()
    dist.destroy_process_group()


CASES = {"gemm": case_gemm, "gemm_bwd": case_gemm_bwd, "skinny_gemm": case_skinny_gemm, "decode_attention": case_decode_attention, "linear_logprob": case_linear_logprob, "linear_sample": case_linear_sample,
         "elementwise": case_elementwise, "peer": case_peer, "decode_step": case_decode_step, "train_step": case_train_step, "attention": case_attention}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="18800x6144x2560,18800x2560x4096,18800x19456x2560,18800x2560x9728,8192x8192x8192", help="gemm: MxNxK list")
    ap.add_argument("--skinny-shapes", default="", help="skinny_gemm: MxNxK list")
    ap.add_argument("--no-library", action="store_true", help="gemm: skip the library GEMM (for profiler captures)")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=2688)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=18800)
    ap.add_argument("--hidden", type=int, default=2560)
    ap.add_argument("--intermediate", type=int, default=9728)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--ragged", action="store_true", help="attention: do not pass host sequence lengths")
    ap.add_argument("--seqs", type=int, default=4, help="train_step: sequences per micro-batch")
    ap.add_argument("--layers", type=int, default=0, help="decode_step: number of decoder blocks (0 = the full 36)")
    ap.add_argument("--numel", type=int, default=101_000_000, help="peer: parameters in one sharded group (a Qwen3-4B block has 101 M)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    CASES[args.case](args)


if __name__ == "__main__":
    main()
