"""Batched autoregressive generation over a paged KV cache with a host-free decode step.

Per wave of sequences:

1. pages for ``prompt + max_new_tokens`` are reserved up front, so block tables are static;
2. prompts are prefilled *packed* (no padding) in token-budgeted chunks;
3. the decode step — embed, N layers with paged attention, final norm, lm_head, sampler, and the
   bookkeeping (append token/log-prob at column ``t``, advance positions / lengths / slots, latch
   the finished flag on EOS) — touches only device tensors.  On CUDA it is captured once per
   batch size into a CUDA graph and replayed; the host merely polls an "all finished" flag every
   ``poll_interval`` steps, replacing the reference's per-token ``all_reduce(MIN)`` barrier
   (``unirl/models/qwen3/ar.py:318-321``).

The sampler records the temperature-scaled *full-softmax* log-prob (before top-k/top-p
truncation), which is exactly what the trainer's replay recomputes.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from unirl_b200.models.qwen3.modeling import AttnMeta
from unirl_b200.ops import sampling as S
from unirl_b200.rollout.engine.native_ar.kv_cache import PagedKVCache


@dataclass
class GenerationOutput:
    tokens: List[torch.Tensor]  # per sequence [n_i] int64
    log_probs: List[torch.Tensor]  # per sequence [n_i] fp32
    finished: torch.Tensor  # [B] bool: stopped on EOS (False ⇒ truncated at max_new_tokens)
    num_steps: int = 0


class ARGenerator:
    def __init__(self, model: Any, *, page_size: int = 64, max_running: int = 256, prefill_token_budget: int = 16384,
                 kv_cache_tokens: Optional[int] = None, use_cuda_graph: bool = True, poll_interval: int = 64, seed: int = 0,
                 cache_dtype: Optional[torch.dtype] = None, share_prefix: bool = True):
        self.model = model
        self.share_prefix = bool(share_prefix)  # samples of one prompt share its KV pages and read them once per decode step
        self.cfg = model.cfg
        self.page_size, self.max_running = int(page_size), int(max_running)
        self.prefill_token_budget = int(prefill_token_budget)
        self.kv_cache_tokens = kv_cache_tokens
        self.poll_interval = int(poll_interval)
        self.seed = int(seed)
        self.device = model.embed_tokens.device
        self.use_cuda_graph = bool(use_cuda_graph) and self.device.type == "cuda"
        self.cache_dtype = cache_dtype or model.embed_tokens.dtype
        self.cache: Optional[PagedKVCache] = None
        self._graphs: Dict[Tuple[int, int, float, int, float], Any] = {}
        self._calls = 0

    # ---- memory -----------------------------------------------------------------------------------
    def ensure_cache(self, tokens_needed: int) -> PagedKVCache:
        pages = math.ceil(tokens_needed / self.page_size) + 1
        if self.kv_cache_tokens is not None:
            pages = max(pages, math.ceil(self.kv_cache_tokens / self.page_size))
        if self.cache is None or self.cache.num_pages < pages:
            self.release_cache()
            layer0 = self.model.layers[0]
            self.cache = PagedKVCache(self.cfg.num_hidden_layers, layer0.n_kv, self.cfg.head_dim, self.page_size, pages, self.cache_dtype, self.device)
        elif not self.cache.is_allocated:
            self.cache.allocate()
        return self.cache

    def release_cache(self) -> None:
        self._graphs.clear()
        if self.cache is not None:
            self.cache.release()
        self.cache = None

    # ---- public -------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[torch.Tensor], *, max_new_tokens: int, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, stop_token_ids: Optional[Sequence[int]] = None, seed: Optional[int] = None,
                 extras: Optional[Sequence[Any]] = None) -> GenerationOutput:
        """``prompts``: per-sequence 1-D token tensors.  Sequences beyond ``max_running`` run in successive waves.

        ``extras``: optional per-sequence multimodal payloads handed to ``model.prepare_multimodal`` at prefill (a
        vision-language model merges image features into the prompt embeddings and returns 3-axis rotary positions plus
        the per-sequence offset its decode positions carry)."""
        n = len(prompts)
        toks: List[Optional[torch.Tensor]] = [None] * n
        lps: List[Optional[torch.Tensor]] = [None] * n
        fin = torch.zeros(n, dtype=torch.bool)
        steps = 0
        seed = self.seed + self._calls if seed is None else int(seed)
        self._calls += 1
        for lo in range(0, n, self.max_running):
            idx = list(range(lo, min(n, lo + self.max_running)))
            t, l, f, s = self._run_wave([prompts[i] for i in idx], max_new_tokens, temperature, top_k, top_p, stop_token_ids, seed + lo,
                                        None if extras is None else [extras[i] for i in idx])
            for j, i in enumerate(idx):
                toks[i], lps[i] = t[j], l[j]
            fin[lo : lo + len(idx)] = f
            steps += s
        return GenerationOutput(toks, lps, fin, steps)  # type: ignore[arg-type]

    # ---- one wave -------------------------------------------------------------------------------------
    def _run_wave(self, prompts: List[torch.Tensor], max_new: int, temperature: float, top_k: int, top_p: float,
                  stop_ids: Optional[Sequence[int]], seed: int, extras: Optional[List[Any]] = None):
        dev, ps, b = self.device, self.page_size, len(prompts)
        rope_offset = torch.zeros(b, dtype=torch.long, device=dev)
        plens = [int(p.numel()) for p in prompts]
        rows = self._shared_rows(prompts) if (extras is None and dev.type == "cuda" and self.share_prefix) else 1
        shared_pages = [(pl // ps if rows > 1 else 0) for pl in plens]  # whole pages of the prompt, shared inside a chunk of `rows` samples
        own_pages = [math.ceil((pl - sp * ps + max_new) / ps) for pl, sp in zip(plens, shared_pages)]
        total_pages = sum(own_pages) + sum(shared_pages[i] for i in range(0, b, rows))
        cache = self.ensure_cache(total_pages * ps)
        cache.allocator.reset()
        max_pages = max(s_ + o for s_, o in zip(shared_pages, own_pages))
        bt = torch.zeros(b, max_pages, dtype=torch.int32)
        pre_t = torch.zeros(max(1, b // rows), max(1, max(shared_pages)), dtype=torch.int32)
        suf_t = torch.zeros(b, max(own_pages), dtype=torch.int32)
        for i in range(b):
            if i % rows == 0:
                lead = torch.tensor(cache.allocator.allocate(shared_pages[i]), dtype=torch.int32) if shared_pages[i] else torch.zeros(0, dtype=torch.int32)
                pre_t[i // rows, : shared_pages[i]] = lead
            own = torch.tensor(cache.allocator.allocate(own_pages[i]), dtype=torch.int32)
            bt[i, : shared_pages[i]] = lead
            bt[i, shared_pages[i] : shared_pages[i] + own_pages[i]] = own
            suf_t[i, : own_pages[i]] = own
        block_tables = bt.to(dev)
        stop = torch.tensor(list(stop_ids) if stop_ids else [self.cfg.eos_token_id], dtype=torch.long, device=dev)

        # -- prefill (packed, chunked by token budget) --------------------------------------------------
        last_hidden = torch.empty(b, self.cfg.hidden_size, dtype=self.model.embed_tokens.dtype, device=dev)
        leaders = list(range(0, b, rows))  # with shared prefixes only the first sample of a chunk runs the prompt
        i = 0
        while i < len(leaders):
            j, tot = i, 0
            while j < len(leaders) and (j == i or tot + plens[leaders[j]] <= self.prefill_token_budget):
                tot += plens[leaders[j]]
                j += 1
            idx = leaders[i:j]
            sel = torch.tensor(idx, device=dev)
            out = torch.empty(len(idx), self.cfg.hidden_size, dtype=last_hidden.dtype, device=dev)
            deltas = torch.zeros(len(idx), dtype=torch.long, device=dev) if rows == 1 else None  # advanced indexing copies: collect, then scatter
            self._prefill([prompts[k] for k in idx], [plens[k] for k in idx], block_tables[sel], cache, out,
                          None if extras is None else [extras[k] for k in idx], deltas)
            if deltas is not None:
                rope_offset[sel] = deltas
            last_hidden[sel] = out
            i = j
        if rows > 1:
            # followers: same last hidden state; the prompt's tail (the tokens past its last whole page) lives in the leader's first own page
            lead_of = torch.arange(b, device=dev) // rows * rows
            last_hidden.copy_(last_hidden[lead_of])
            follow = [k for k in range(b) if k % rows and plens[k] % ps]
            if follow:
                src = torch.tensor([int(suf_t[k // rows * rows, 0]) for k in follow], device=dev)
                dst = torch.tensor([int(suf_t[k, 0]) for k in follow], device=dev)
                for layer_k, layer_v in zip(cache.k, cache.v):
                    layer_k[dst] = layer_k[src]
                    layer_v[dst] = layer_v[src]

        # -- decode state (all device resident) ---------------------------------------------------------
        st = _DecodeState(b, max_new, dev)
        st.positions.copy_(torch.tensor(plens, dtype=torch.long))  # index at which the next fed token is written
        st.rope_offset.copy_(rope_offset)
        first_tok, first_lp = self._sample(last_hidden, temperature, top_k, top_p, seed, 0, st)
        st.record(first_tok, first_lp, stop)
        meta = AttnMeta(mode="decode", positions=st.rope_pos, k_cache=cache.k, v_cache=cache.v, block_tables=block_tables,
                        seq_lens=st.seq_lens, slot_mapping=st.slots, max_kv_len=max(plens) + max_new)
        if self.device.type == "cuda":
            from unirl_b200.ops._ext import ext

            C = ext()
            layer0 = self.model.layers[0]
            if rows > 1 and C is not None:
                from types import SimpleNamespace

                st.prefix_len = torch.tensor([shared_pages[k] * ps for k in range(b)], dtype=torch.int32, device=dev)
                st.suffix_lens = torch.zeros(b, dtype=torch.int32, device=dev)
                meta.cascade = SimpleNamespace(prefix_tables=pre_t.to(dev), prefix_lens=st.prefix_len[::rows].contiguous(), suffix_tables=suf_t.to(dev),
                                               suffix_lens=st.suffix_lens, rows=rows)
                meta.workspace = torch.empty(C.decode_cascade_workspace_size(b, rows, layer0.n_q, layer0.n_kv, self.cfg.head_dim, meta.max_kv_len),
                                             dtype=torch.float32, device=dev)
            elif C is not None and hasattr(C, "decode_workspace_size"):
                meta.workspace = torch.empty(C.decode_workspace_size(b, layer0.n_q, self.cfg.head_dim, meta.max_kv_len), dtype=torch.float32, device=dev)

        def step() -> None:
            st.prepare(block_tables, ps)
            hidden = self.model(st.cur_tokens, meta)
            tok, lp = self._sample(hidden, temperature, top_k, top_p, seed, None, st)
            st.record(tok, lp, stop)
            st.positions.add_(1)

        n_steps = 1
        if max_new > 1:
            step()  # first decode step runs eagerly: one-time kernel attribute / library workspace set-up must not happen under capture
            n_steps = 2
        runner = self._graphed(step, b, max_new, temperature, top_k, top_p) if self.use_cuda_graph and max_new > 2 else step
        while n_steps < max_new:
            burst = min(self.poll_interval, max_new - n_steps)
            for _ in range(burst):
                runner()
            n_steps += burst
            if bool(st.finished.all()):  # one small D2H read per `poll_interval` steps
                break
        lens = st.lengths.cpu()
        out_t, out_l = st.out_tokens.cpu(), st.out_logp.cpu()
        toks = [out_t[k, : int(lens[k])].clone() for k in range(b)]
        lps = [out_l[k, : int(lens[k])].clone() for k in range(b)]
        return toks, lps, st.finished.cpu(), n_steps

    def _shared_rows(self, prompts: List[torch.Tensor]) -> int:
        """How many consecutive sequences can share a prefix job: the largest R in {4, 2} such that the batch is made of chunks of R
        identical prompts and R query-head groups fit the 16-row attention tile; 1 when nothing repeats."""
        b = len(prompts)
        gs = self.model.layers[0].n_q // self.model.layers[0].n_kv
        for r in (4, 2):
            if r * gs > 16 or b % r:
                continue
            if all(prompts[i].numel() == prompts[i - i % r].numel() and bool(torch.equal(prompts[i], prompts[i - i % r])) for i in range(b) if i % r):
                return r
        return 1

    def _prefill(self, prompts: List[torch.Tensor], plens: List[int], block_tables: torch.Tensor, cache: PagedKVCache, out_last: torch.Tensor,
                 extras: Optional[List[Any]] = None, rope_offset_out: Optional[torch.Tensor] = None) -> None:
        dev, ps = self.device, self.page_size
        tokens = torch.cat([p.to(torch.long) for p in prompts]).to(dev)
        cu = torch.zeros(len(plens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(plens, dtype=torch.int32).cumsum(0)
        positions = torch.cat([torch.arange(n) for n in plens]).to(dev)
        seq_id = torch.repeat_interleave(torch.arange(len(plens)), torch.tensor(plens)).to(dev)
        page = block_tables[seq_id, (positions // ps)].long()
        meta = AttnMeta(mode="prefill", positions=positions, cu_seqlens=cu.to(dev), max_seqlen=max(plens), k_cache=cache.k, v_cache=cache.v,
                        slot_mapping=page * ps + positions % ps, seq_lens_host=list(plens))
        if extras is not None and hasattr(self.model, "prepare_multimodal"):
            deltas = self.model.prepare_multimodal(prompts, extras, meta)
            if rope_offset_out is not None and deltas is not None:
                rope_offset_out.copy_(deltas.to(rope_offset_out))
        hidden = self.model(tokens, meta)
        out_last.copy_(hidden[(cu[1:].long() - 1).to(dev)])

    def _sample(self, hidden: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, step: Optional[int], st: "_DecodeState"):
        """Vocab projection + sampling of the last hidden states (fused on CUDA; see ``ops.sampling.linear_sample``)."""
        w = self.model.output_weight
        if hidden.is_cuda:
            return S.linear_sample(hidden, w, temperature, top_k, top_p, seed=seed, step=0 if step is None else step, step_tensor=st.step_counter)
        if st.cpu_gen is None:
            st.cpu_gen = torch.Generator().manual_seed(seed)
        return S.sample_reference(torch.nn.functional.linear(hidden, w), temperature, top_k, top_p, st.cpu_gen)

    def _graphed(self, step_fn, b: int, max_new: int, temperature: float, top_k: int, top_p: float):
        """Capture ``step_fn`` (which closes over this wave's state tensors) into a CUDA graph."""
        fused = getattr(getattr(self.model, "tp", None), "fused", None)  # peer-memory all-reduce: replay must start on staging half 0
        if fused is not None:
            fused.align()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        from unirl_b200.ops._ext import count_launch, launch_count

        g = torch.cuda.CUDAGraph()
        n0 = launch_count()
        # capture itself does not execute the step, so the decode state is not advanced here
        with torch.cuda.graph(g, stream=s):
            step_fn()
            if fused is not None:
                fused.align()
        per_replay = launch_count() - n0  # native kernels recorded in the graph: every replay launches them again
        self._graphs[(b, max_new, temperature, top_k, top_p)] = g  # keep alive for the wave

        def replay() -> None:
            g.replay()
            count_launch(per_replay)

        return replay


class _DecodeState:
    """Device-resident per-wave decode bookkeeping (mutated in place so a CUDA graph can own it)."""

    def __init__(self, b: int, max_new: int, dev: torch.device):
        z = lambda dt, *shape: torch.zeros(*shape, dtype=dt, device=dev)  # noqa: E731
        self.out_tokens, self.out_logp = z(torch.long, b, max_new), z(torch.float32, b, max_new)
        self.cur_tokens, self.positions, self.slots = z(torch.long, b), z(torch.long, b), z(torch.long, b)
        self.prefix_len: Optional[torch.Tensor] = None  # shared-prefix decode: tokens of each sequence that live in shared pages
        self.suffix_lens: Optional[torch.Tensor] = None
        self.rope_offset, self.rope_pos = z(torch.long, b), z(torch.long, b)  # rotary position = cache index + per-sequence offset
        self.seq_lens = z(torch.int32, b)
        self.lengths = z(torch.long, b)
        self.finished = z(torch.bool, b)
        self.step_counter = z(torch.long, 1)
        self.rows = torch.arange(b, device=dev)
        self.max_new = max_new
        self.cpu_gen: Optional[torch.Generator] = None

    def record(self, tok: torch.Tensor, lp: torch.Tensor, stop: torch.Tensor) -> None:
        """Append the sampled token for every unfinished row, then latch EOS."""
        live = ~self.finished
        col = self.lengths.clamp(max=self.max_new - 1)
        self.out_tokens[self.rows, col] = torch.where(live, tok, self.out_tokens[self.rows, col])
        self.out_logp[self.rows, col] = torch.where(live, lp.float(), self.out_logp[self.rows, col])
        self.lengths.add_(live.long())
        self.cur_tokens.copy_(tok)
        self.finished.logical_or_((tok.unsqueeze(1) == stop.unsqueeze(0)).any(1))
        self.finished.logical_or_(self.lengths >= self.max_new)
        self.step_counter.add_(1)

    def prepare(self, block_tables: torch.Tensor, page_size: int) -> None:
        """``positions[b]`` is the index of the token fed this step: derive its cache slot and the KV length."""
        page = block_tables.gather(1, (self.positions // page_size).unsqueeze(1)).squeeze(1).long()
        self.slots.copy_(page * page_size + self.positions % page_size)
        self.seq_lens.copy_((self.positions + 1).to(torch.int32))
        self.rope_pos.copy_(self.positions + self.rope_offset)
        if self.suffix_lens is not None:
            self.suffix_lens.copy_(self.seq_lens - self.prefix_len)


__all__ = ["ARGenerator", "GenerationOutput"]
