"""Batched autoregressive generation over a paged KV cache with a host-free decode step.

Scheduling is continuous (``continuous=True``, the default): up to ``max_running`` sequences decode together; every
``poll_interval`` steps the host reads the finished flags, retires finished sequences (their pages go back to the allocator),
admits queued prompts into the freed rows (chunked prefill) and -- once nothing is queued -- compacts the live rows to the front
and switches to the CUDA graph of a smaller batch-size bucket, so the number of decode steps follows the sum of the response
lengths instead of (longest response) x (number of waves).  The random stream of a sequence is keyed on (sequence index, token
index), so its draws do not depend on where or when it runs.  Reference behaviour replaced: one request per sample handed to the
serving engine's continuous batching (``unirl/rollout/engine/sglang_llm/engine.py:373-581``).

``continuous=False`` keeps fixed waves.  Per wave of sequences:

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

import os

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
                 cache_dtype: Optional[torch.dtype] = None, share_prefix: bool = True, continuous: bool = True):
        self.model = model
        self.continuous = bool(continuous)
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
        if self.continuous and n:
            t, l, f, steps = self._run_continuous(list(prompts), max_new_tokens, temperature, top_k, top_p, stop_token_ids, seed,
                                                  None if extras is None else list(extras))
            return GenerationOutput(t, l, f, steps)
        for lo in range(0, n, self.max_running):
            idx = list(range(lo, min(n, lo + self.max_running)))
            t, l, f, s = self._run_wave([prompts[i] for i in idx], max_new_tokens, temperature, top_k, top_p, stop_token_ids, seed,
                                        None if extras is None else [extras[i] for i in idx], first_id=lo)
            for j, i in enumerate(idx):
                toks[i], lps[i] = t[j], l[j]
            fin[lo : lo + len(idx)] = f
            steps += s
        return GenerationOutput(toks, lps, fin, steps)  # type: ignore[arg-type]

    # ---- one wave -------------------------------------------------------------------------------------
    def _run_wave(self, prompts: List[torch.Tensor], max_new: int, temperature: float, top_k: int, top_p: float,
                  stop_ids: Optional[Sequence[int]], seed: int, extras: Optional[List[Any]] = None, first_id: int = 0):
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
        st.rng_ids.add_(first_id)  # random streams are keyed on the sequence's index in the whole call
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
            st.record(tok, lp, stop, fuse_advance=True)
            st.advance()

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
        stop_set = {int(x) for x in stop.tolist()}
        done = torch.tensor([bool(int(lens[k])) and int(toks[k][-1]) in stop_set for k in range(b)], dtype=torch.bool)  # False: cut at max_new_tokens
        return toks, lps, done, n_steps

    # ---- continuous batching ----------------------------------------------------------------------------
    def _run_continuous(self, prompts: List[torch.Tensor], max_new: int, temperature: float, top_k: int, top_p: float,
                        stop_ids: Optional[Sequence[int]], seed: int, extras: Optional[List[Any]] = None):
        """All sequences of the call through one running batch of at most ``max_running`` rows (see the module docstring).

        Sequences are scheduled in *groups*: ``rows`` consecutive samples of one prompt that share its KV pages (1 without sharing).
        A group holds ``rows`` adjacent batch rows from admission until all its members have finished."""
        from collections import deque

        dev, ps, n = self.device, self.page_size, len(prompts)
        plens = [int(p.numel()) for p in prompts]
        rows = self._shared_rows(prompts) if (extras is None and dev.type == "cuda" and self.share_prefix) else 1
        n_groups = n // rows
        cap_g = max(1, min(n_groups, self.max_running // rows))
        cap = cap_g * rows
        shared_pages = [(pl // ps if rows > 1 else 0) for pl in plens]
        own_pages = [math.ceil((pl - sp * ps + max_new) / ps) for pl, sp in zip(plens, shared_pages)]
        group_pages = [shared_pages[g * rows] + sum(own_pages[g * rows : (g + 1) * rows]) for g in range(n_groups)]
        cache = self.ensure_cache((sum(sorted(group_pages, reverse=True)[:cap_g]) + 1) * ps)
        cache.allocator.reset()
        scratch = int(cache.allocator.allocate(1)[0])  # rows without a sequence point here: their (ignored) KV writes touch no live page
        max_pages = max(s_ + o for s_, o in zip(shared_pages, own_pages))
        w_pre, w_suf = max(1, max(shared_pages)), max(own_pages)
        bt_host = torch.full((cap, max_pages), scratch, dtype=torch.int32)
        pre_host = torch.full((cap_g, w_pre), scratch, dtype=torch.int32)
        suf_host = torch.full((cap, w_suf), scratch, dtype=torch.int32)
        block_tables, pre_t, suf_t = bt_host.to(dev), pre_host.to(dev), suf_host.to(dev)
        stop = torch.tensor(list(stop_ids) if stop_ids else [self.cfg.eos_token_id], dtype=torch.long, device=dev)
        stop_set = {int(x) for x in stop.tolist()}

        st = _DecodeState(cap, max_new, dev)
        st.finished.fill_(True)  # every row starts empty
        cascade = rows > 1 and dev.type == "cuda"
        if cascade:
            st.prefix_len = torch.zeros(cap, dtype=torch.int32, device=dev)
            st.suffix_lens = torch.zeros(cap, dtype=torch.int32, device=dev)
        prefix_len_g = torch.zeros(cap_g, dtype=torch.int32, device=dev)
        max_kv = max(plens) + max_new
        C = None
        if dev.type == "cuda":
            from unirl_b200.ops._ext import ext

            C = ext()
        layer0 = self.model.layers[0]

        toks: List[Optional[torch.Tensor]] = [None] * n
        lps: List[Optional[torch.Tensor]] = [None] * n
        fin_out = torch.zeros(n, dtype=torch.bool)
        pending = deque(range(n_groups))
        slot_group: List[Optional[int]] = [None] * cap_g  # group held by every group-slot
        slot_pages: List[List[int]] = [[] for _ in range(cap_g)]

        def admit(slots: List[int]) -> None:
            """Give each listed free group-slot the next queued group: pages, prefill, first token."""
            groups = [pending.popleft() for _ in slots]
            new_rows: List[int] = []
            for slot, g in zip(slots, groups):
                lead_seq = g * rows
                lead = cache.allocator.allocate(shared_pages[lead_seq]) if shared_pages[lead_seq] else []
                held = list(lead)
                pre_host[slot].fill_(scratch)
                if lead:
                    pre_host[slot, : len(lead)] = torch.tensor(lead, dtype=torch.int32)
                for j in range(rows):
                    seq, row = lead_seq + j, slot * rows + j
                    own = cache.allocator.allocate(own_pages[seq])
                    held += list(own)
                    bt_host[row].fill_(scratch)
                    suf_host[row].fill_(scratch)
                    if lead:
                        bt_host[row, : len(lead)] = torch.tensor(lead, dtype=torch.int32)
                    bt_host[row, len(lead) : len(lead) + len(own)] = torch.tensor(own, dtype=torch.int32)
                    suf_host[row, : len(own)] = torch.tensor(own, dtype=torch.int32)
                    new_rows.append(row)
                slot_group[slot], slot_pages[slot] = g, held
            rsel = torch.tensor(new_rows, device=dev)
            gsel = torch.tensor(slots, device=dev)
            block_tables[rsel] = bt_host[new_rows].to(dev)
            suf_t[rsel] = suf_host[new_rows].to(dev)
            pre_t[gsel] = pre_host[slots].to(dev)
            # prefill the group leaders, packed, in token-budgeted chunks
            seq_of_row = [slot_group[r // rows] * rows + r % rows for r in new_rows]  # type: ignore[operator]
            leaders = [k for k in range(len(new_rows)) if new_rows[k] % rows == 0]
            hidden_new = torch.empty(len(new_rows), self.cfg.hidden_size, dtype=self.model.embed_tokens.dtype, device=dev)
            offsets = torch.zeros(len(new_rows), dtype=torch.long, device=dev)
            i = 0
            while i < len(leaders):
                j, tot = i, 0
                while j < len(leaders) and (j == i or tot + plens[seq_of_row[leaders[j]]] <= self.prefill_token_budget):
                    tot += plens[seq_of_row[leaders[j]]]
                    j += 1
                ks = leaders[i:j]
                out = torch.empty(len(ks), self.cfg.hidden_size, dtype=hidden_new.dtype, device=dev)
                deltas = torch.zeros(len(ks), dtype=torch.long, device=dev) if rows == 1 else None
                self._prefill([prompts[seq_of_row[k]] for k in ks], [plens[seq_of_row[k]] for k in ks], block_tables[rsel[ks]], cache, out,
                              None if extras is None else [extras[seq_of_row[k]] for k in ks], deltas)
                for u in range(rows):  # followers start from their leader's last hidden state
                    hidden_new[torch.tensor([k + u for k in ks], device=dev)] = out
                if deltas is not None:
                    offsets[torch.tensor(ks, device=dev)] = deltas
                i = j
            if rows > 1:
                # the prompt's tail (tokens past its last whole page) lives in the leader's first own page: copy it to the followers
                follow = [k for k in range(len(new_rows)) if new_rows[k] % rows and plens[seq_of_row[k]] % ps]
                if follow:
                    src = torch.tensor([int(suf_host[new_rows[k] // rows * rows, 0]) for k in follow], device=dev)
                    dst = torch.tensor([int(suf_host[new_rows[k], 0]) for k in follow], device=dev)
                    for layer_k, layer_v in zip(cache.k, cache.v):
                        layer_k[dst] = layer_k[src]
                        layer_v[dst] = layer_v[src]
            # row state + first token
            ids = torch.tensor(seq_of_row, dtype=torch.long, device=dev)
            st.positions[rsel] = torch.tensor([plens[q] for q in seq_of_row], dtype=torch.long, device=dev)
            st.rope_offset[rsel] = offsets
            st.lengths[rsel] = 0
            st.rng_ids[rsel] = ids
            if cascade:
                st.prefix_len[rsel] = torch.tensor([shared_pages[q] * ps for q in seq_of_row], dtype=torch.int32, device=dev)
                prefix_len_g[gsel] = torch.tensor([shared_pages[slot_group[sl] * rows] * ps for sl in slots], dtype=torch.int32, device=dev)  # type: ignore[operator]
            w = self.model.output_weight
            if dev.type == "cuda":
                tok, lp = S.linear_sample(hidden_new, w, temperature, top_k, top_p, seed=seed, rng_rows=ids, rng_steps=torch.zeros_like(ids))
            else:
                if st.cpu_gen is None:
                    st.cpu_gen = torch.Generator().manual_seed(seed)
                tok, lp = S.sample_reference(torch.nn.functional.linear(hidden_new, w), temperature, top_k, top_p, st.cpu_gen)
            st.out_tokens[rsel, 0] = tok
            st.out_logp[rsel, 0] = lp.float()
            st.cur_tokens[rsel] = tok
            st.lengths[rsel] = 1
            st.finished[rsel] = (tok.unsqueeze(1) == stop.unsqueeze(0)).any(1) | (max_new <= 1)

        def retire(slot: int) -> None:
            g = slot_group[slot]
            lo = slot * rows
            lens = st.lengths[lo : lo + rows].cpu()
            out_t, out_l = st.out_tokens[lo : lo + rows].cpu(), st.out_logp[lo : lo + rows].cpu()
            for j in range(rows):
                seq = g * rows + j  # type: ignore[operator]
                toks[seq], lps[seq] = out_t[j, : int(lens[j])].clone(), out_l[j, : int(lens[j])].clone()
                fin_out[seq] = bool(int(lens[j])) and int(toks[seq][-1]) in stop_set
            cache.allocator.free(slot_pages[slot])
            slot_group[slot], slot_pages[slot] = None, []
            bt_host[lo : lo + rows].fill_(scratch)
            suf_host[lo : lo + rows].fill_(scratch)
            pre_host[slot].fill_(scratch)
            block_tables[lo : lo + rows] = scratch
            suf_t[lo : lo + rows] = scratch
            pre_t[slot] = scratch
            st.positions[lo : lo + rows] = 0
            if cascade:
                st.prefix_len[lo : lo + rows] = 0
                prefix_len_g[slot] = 0

        def compact(n_live_slots: int) -> None:
            """Move the live group-slots to the front (order kept), so a smaller bucket covers them."""
            live = [sl for sl in range(cap_g) if slot_group[sl] is not None]
            dead = [sl for sl in range(cap_g) if slot_group[sl] is None]
            order = live + dead
            if order == list(range(cap_g)):
                return
            gperm = torch.tensor(order, device=dev)
            rperm = (gperm.unsqueeze(1) * rows + torch.arange(rows, device=dev)).reshape(-1)
            for name in _DecodeState._ROW_FIELDS:
                t = getattr(st, name)
                if t is not None:
                    t.copy_(t[rperm])
            for t in (block_tables, suf_t):
                t.copy_(t[rperm])
            pre_t.copy_(pre_t[gperm])
            prefix_len_g.copy_(prefix_len_g[gperm])
            hperm = rperm.cpu()
            bt_host.copy_(bt_host[hperm])
            suf_host.copy_(suf_host[hperm])
            pre_host.copy_(pre_host[gperm.cpu()])
            slot_group[:] = [slot_group[sl] for sl in order]
            slot_pages[:] = [slot_pages[sl] for sl in order]

        # batch-size buckets: one captured graph each; the running batch only ever shrinks through them
        buckets = sorted({cap} | {b for b in (cap_g >> k for k in range(1, 8)) for b in [b * rows] if b >= max(8, rows) and b < cap}, reverse=True)
        runners: Dict[int, Any] = {}
        ws_floats = 0
        if C is not None:
            for b in buckets:
                ws_floats = max(ws_floats, int(C.decode_cascade_workspace_size(b, rows, layer0.n_q, layer0.n_kv, self.cfg.head_dim, max_kv)) if cascade
                                else int(C.decode_workspace_size(b, layer0.n_q, self.cfg.head_dim, max_kv)))
        workspace = torch.empty(ws_floats, dtype=torch.float32, device=dev) if ws_floats else None

        def runner_for(b: int):
            if b in runners:
                return runners[b]
            v = st.view(b)
            bt_b = block_tables[:b]
            meta = AttnMeta(mode="decode", positions=v.rope_pos, k_cache=cache.k, v_cache=cache.v, block_tables=bt_b, seq_lens=v.seq_lens,
                            slot_mapping=v.slots, max_kv_len=max_kv)
            meta.workspace = workspace
            if cascade:
                from types import SimpleNamespace

                meta.cascade = SimpleNamespace(prefix_tables=pre_t[: b // rows], prefix_lens=prefix_len_g[: b // rows], suffix_tables=suf_t[:b],
                                               suffix_lens=v.suffix_lens, rows=rows)

            def step() -> None:
                v.prepare(bt_b, ps)
                hidden = self.model(v.cur_tokens, meta)
                tok, lp = self._sample(hidden, temperature, top_k, top_p, seed, None, v)
                v.record(tok, lp, stop, fuse_advance=True)
                v.advance()

            step()  # one eager step per bucket: one-time kernel attribute / library workspace set-up must not happen under capture
            runners[b] = self._graphed(step, b, max_new, temperature, top_k, top_p) if self.use_cuda_graph else step
            return runners[b]

        admit(list(range(min(cap_g, len(pending)))))
        b_act, n_steps = cap, 1
        while True:
            live_slots = [sl for sl in range(cap_g) if slot_group[sl] is not None]
            if not live_slots and not pending:
                break
            fresh = b_act not in runners
            run = runner_for(b_act)
            burst = self.poll_interval - (1 if fresh else 0)
            for _ in range(max(0, burst)):
                run()
            n_steps += self.poll_interval
            fin = st.finished[:b_act].cpu().view(-1, rows).all(1)  # the one D2H read per `poll_interval` steps
            freed = [sl for sl in range(b_act // rows) if slot_group[sl] is not None and bool(fin[sl])]
            for sl in freed:
                retire(sl)
            if pending:
                free = [sl for sl in range(b_act // rows) if slot_group[sl] is None][: len(pending)]
                if free:
                    admit(free)
            else:
                n_live = sum(1 for sl in range(cap_g) if slot_group[sl] is not None)
                smaller = [b for b in buckets if b < b_act and b >= n_live * rows]
                if n_live and smaller:
                    compact(n_live)
                    b_act = min(smaller)
        fused = getattr(getattr(self.model, "tp", None), "fused", None)
        if fused is not None:
            fused.align()
        return toks, lps, fin_out, n_steps

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
            return S.linear_sample(hidden, w, temperature, top_k, top_p, seed=seed, step=0 if step is None else step, step_tensor=st.step_counter,
                                   rng_rows=st.rng_ids, rng_steps=st.lengths)
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
        self.rng_ids = torch.arange(b, device=dev)  # sequence index that keys the row's random stream (with `lengths` as the token index)
        self.max_new = max_new
        self.cpu_gen: Optional[torch.Generator] = None
        self._advanced = False

    _ROW_FIELDS = ("out_tokens", "out_logp", "cur_tokens", "positions", "slots", "rope_offset", "rope_pos", "seq_lens", "lengths", "finished", "rng_ids",
                   "prefix_len", "suffix_lens")

    def view(self, b: int) -> "_DecodeState":
        """The first ``b`` rows as a state of their own (tensors are views: a CUDA graph captured on them follows later in-place updates)."""
        v = object.__new__(_DecodeState)
        v.__dict__.update(self.__dict__)
        for name in self._ROW_FIELDS:
            t = getattr(self, name)
            setattr(v, name, None if t is None else t[:b])
        v.rows = self.rows[:b]
        return v

    def advance(self) -> None:
        """Move every LIVE row to its next cache index; a finished row stays where it is (it keeps rewriting one slot of its own pages
        until it is retired, instead of walking past the pages reserved for it)."""
        if self._advanced:  # the fused record kernel already did it
            self._advanced = False
            return
        self.positions.add_((~self.finished).long())

    def _native(self) -> Any:
        if not self.positions.is_cuda:
            return None
        from unirl_b200.ops._ext import ext

        C = ext()
        if os.environ.get("UNIRL_B200_DECODE_BOOKKEEPING", "1") == "0":  # A/B switch: the element-wise composition
            return None
        return C if C is not None and hasattr(C, "decode_record_advance") else None

    def record(self, tok: torch.Tensor, lp: torch.Tensor, stop: torch.Tensor, fuse_advance: bool = False) -> None:
        """Append the sampled token for every unfinished row, then latch EOS.  On CUDA one kernel does this and (``fuse_advance``) the
        advance of the cache index that follows it in the decode step."""
        C = self._native() if fuse_advance else None
        if C is not None:
            from unirl_b200.ops._ext import count_launch

            C.decode_record_advance(tok.contiguous(), lp.float().contiguous(), stop.contiguous(), self.out_tokens, self.out_logp, self.cur_tokens, self.lengths,
                                    self.finished, self.positions, self.step_counter)
            count_launch()
            self._advanced = True
            return
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
        """``positions[b]`` is the index of the token fed this step: derive its cache slot and the KV length (one kernel on CUDA)."""
        C = self._native()
        if C is not None and block_tables.dtype == torch.int32:
            from unirl_b200.ops._ext import count_launch

            C.decode_prepare(self.positions, block_tables, int(page_size), self.rope_offset, self.slots, self.seq_lens, self.rope_pos, self.prefix_len, self.suffix_lens)
            count_launch()
            return
        page = block_tables.gather(1, (self.positions // page_size).unsqueeze(1)).squeeze(1).long()
        self.slots.copy_(page * page_size + self.positions % page_size)
        self.seq_lens.copy_((self.positions + 1).to(torch.int32))
        self.rope_pos.copy_(self.positions + self.rope_offset)
        if self.suffix_lens is not None:
            self.suffix_lens.copy_(self.seq_lens - self.prefix_len)


__all__ = ["ARGenerator", "GenerationOutput"]
