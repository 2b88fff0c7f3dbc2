"""Qwen3 AR stage: batched generation and teacher-forced log-prob replay.

``replay`` packs ``prompt_i ⊕ response_i`` for the whole micro-batch into ONE unpadded token
stream, runs the decoder body once (varlen attention), gathers the hidden states that predict
response tokens and hands them to the fused ``linear_logprob`` op (lm_head GEMM + log-softmax +
gather, ``[tokens, vocab]`` never materialised).  The reference re-pads to ``[B, L]`` and chunks the
lm_head under activation checkpointing (``unirl/models/qwen3/ar.py:39-99``, ``:330-447``).

``autoregress`` drives :class:`ARGenerator` (paged KV, host-free decode step) on the *same*
module, which is the trainside rollout path; sampling records the full-softmax log-prob before
truncation (``:138-175``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from unirl_b200.models.qwen3.conditions import Qwen3ARConditions
from unirl_b200.models.qwen3.modeling import AttnMeta
from unirl_b200.models.types.contracts import unpad_prompts
from unirl_b200.ops.logprob import linear_logprob
from unirl_b200.ops.sampling import sample_reference
from unirl_b200.types.sampling import ARSamplingParams
from unirl_b200.types.segments import SegmentStatus, TextSegment


@dataclass
class Qwen3ARParams:
    max_tokens: int = 512
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0


class Qwen3ARStep:
    """Per-step sampler: temperature → (top-k, top-p) → multinomial; log-prob taken before truncation."""

    def __init__(self, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, generator: Optional[torch.Generator] = None):
        self.temperature, self.top_k, self.top_p, self.generator = float(temperature), int(top_k), float(top_p), generator

    def step(self, logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return sample_reference(logits, self.temperature, self.top_k, self.top_p, self.generator)


def pack_text_segment(tokens: Sequence[torch.Tensor], log_probs: Sequence[torch.Tensor], finished: torch.Tensor) -> TextSegment:
    status = torch.where(finished.bool(), torch.tensor(int(SegmentStatus.COMPLETED)), torch.tensor(int(SegmentStatus.TRUNCATED)))
    return TextSegment.pack(tokens=[t.to(torch.long).cpu() for t in tokens], log_probs=[l.float().cpu() for l in log_probs],
                            loss_mask=[torch.ones(int(t.numel()), dtype=torch.float32) for t in tokens], status=status.to(torch.long))


_pack_text_segment = pack_text_segment


def build_replay_batch(prompts: List[torch.Tensor], responses: List[torch.Tensor], device: Any):
    """Concatenate ``prompt_i ⊕ response_i`` and index the positions whose *next* token is a response token.

    Returns ``(tokens [T], positions [T], cu_seqlens [B+1] int32, max_len, pred_index [R], targets [R])`` with
    ``R = Σ len(response_i)``, ordered like the packed segment.
    """
    toks, pos, pred, lens = [], [], [], []
    off = 0
    for p, r in zip(prompts, responses):
        n_p, n_r = int(p.numel()), int(r.numel())
        toks += [p.to(torch.long), r.to(torch.long)]
        pos.append(torch.arange(n_p + n_r))
        if n_r:
            pred.append(torch.arange(off + n_p - 1, off + n_p + n_r - 1))
        off += n_p + n_r
        lens.append(n_p + n_r)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    tokens = torch.cat(toks).to(device) if toks else torch.zeros(0, dtype=torch.long, device=device)
    targets = torch.cat([r.to(torch.long) for r in responses]).to(device) if responses else tokens[:0]
    pred_index = torch.cat(pred).to(device) if pred else torch.zeros(0, dtype=torch.long, device=device)
    return tokens, torch.cat(pos).to(device), cu.to(device), max(lens, default=0), pred_index, targets


class Qwen3ARStage:
    def __init__(self, bundle: Any, autocast_precision: str = "bf16", logprob_precision: str = "fp32", generator_kwargs: Optional[dict] = None):
        self.model = bundle
        self.autocast_precision, self.logprob_precision = autocast_precision, logprob_precision
        self.generator_kwargs = dict(generator_kwargs or {})
        self._gen = None

    def trainable_module(self) -> torch.nn.Module:
        return self.model.transformer

    @property
    def generator(self):
        if self._gen is None:
            from unirl_b200.rollout.engine.native_ar.generator import ARGenerator

            self._gen = ARGenerator(self.model.transformer, **self.generator_kwargs)
        return self._gen

    def _resolve_stop_ids(self, sampling_params: ARSamplingParams) -> List[int]:
        ids = {int(self.model.transformer.cfg.eos_token_id)}
        tok_eos = getattr(self.model.tokenizer, "eos_token_id", None)
        if tok_eos is not None:
            ids.add(int(tok_eos))
        if sampling_params.stop_token_id is not None:
            ids.add(int(sampling_params.stop_token_id))
        return sorted(ids)

    def autoregress(self, conditions: Qwen3ARConditions, *, sampling_params: ARSamplingParams, **_kw: Any) -> TextSegment:
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        was_training = self.model.transformer.training
        self.model.transformer.eval()
        try:
            out = self.generator.generate(prompts, max_new_tokens=int(sampling_params.max_new_tokens), temperature=float(sampling_params.temperature),
                                          top_k=int(sampling_params.top_k or 0), top_p=float(sampling_params.top_p),
                                          stop_token_ids=self._resolve_stop_ids(sampling_params))
        finally:
            self.model.transformer.train(was_training)
        return pack_text_segment(out.tokens, out.log_probs, out.finished)

    def replay(self, conditions: Qwen3ARConditions, *, segment: TextSegment, temperature: float = 1.0) -> torch.Tensor:
        if conditions.prompt is None or conditions.prompt.input_ids is None or conditions.prompt.attention_mask is None:
            raise ValueError("Qwen3ARStage.replay: conditions.prompt needs input_ids and attention_mask")
        if segment.tokens is None or segment.cu_seqlens is None:
            raise ValueError("Qwen3ARStage.replay: segment needs packed tokens (build with TextSegment.pack)")
        model = self.model.transformer
        device = model.embed_tokens.device
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        cu = segment.cu_seqlens.tolist()
        responses = [segment.tokens[cu[i] : cu[i + 1]] for i in range(len(cu) - 1)]
        if len(prompts) != len(responses):
            raise ValueError(f"replay: {len(prompts)} prompts vs {len(responses)} responses")
        cp = getattr(model, "cp", None)
        if cp is not None and cp.size > 1:
            return self._replay_context_parallel(prompts, responses, cp, float(temperature))
        tokens, positions, cu_dev, max_len, pred_index, targets = build_replay_batch(prompts, responses, device)
        if not targets.numel():
            return torch.zeros(0, dtype=torch.float32, device=device)
        lens = [int(p.numel()) + int(r.numel()) for p, r in zip(prompts, responses)]
        hidden = model(tokens, AttnMeta(mode="train", positions=positions, cu_seqlens=cu_dev, max_seqlen=max_len, seq_lens_host=lens))
        return linear_logprob(hidden.index_select(0, pred_index), model.output_weight, targets, float(temperature))

    def _replay_context_parallel(self, prompts: List[torch.Tensor], responses: List[torch.Tensor], cp: Any, temperature: float) -> torch.Tensor:
        """Replay with every sequence cut over the context-parallel ranks: this rank runs the model on its chunk of each sequence (keys and
        values gathered per layer), takes the log-probs of the response tokens it holds, and the ranks' pieces are summed into the full
        vector, ordered like the packed segment, so the caller sees what the single-rank replay returns."""
        from unirl_b200.parallel.context_parallel import PackedPlan, _SumOverRanks

        model = self.model.transformer
        device = model.embed_tokens.device
        seqs = [torch.cat([p.to(torch.long).cpu(), r.to(torch.long).cpu()]) for p, r in zip(prompts, responses)]
        plan = PackedPlan([int(s.numel()) for s in seqs], cp.size, cp.rank)
        total = sum(int(r.numel()) for r in responses)
        if not total:
            return torch.zeros(0, dtype=torch.float32, device=device)
        tokens = torch.cat([plan.local_slice(s, i) for i, s in enumerate(seqs)]).to(device)
        meta = AttnMeta(mode="train", positions=plan.local_positions().to(device), cu_seqlens=plan.cu_q.to(device), max_seqlen=max(plan.chunk), cp_plan=plan, cp_comm=cp.comm)
        hidden = model(tokens, meta)
        rows, dest, tgt, off = [], [], [], 0
        for i, (p, r) in enumerate(zip(prompts, responses)):
            n_p, n_r = int(p.numel()), int(r.numel())
            if n_r:
                pred = torch.arange(n_p - 1, n_p + n_r - 1)  # position j predicts token j + 1
                mine, local = plan.locate(i, pred)
                rows.append(local)
                dest.append(torch.arange(off, off + n_r)[mine])
                tgt.append(seqs[i][pred[mine] + 1])
            off += n_r
        rows_t, dest_t, tgt_t = torch.cat(rows).to(device), torch.cat(dest).to(device), torch.cat(tgt).to(device)
        full = torch.zeros(total, dtype=torch.float32, device=device)
        if rows_t.numel():
            full = full.index_put((dest_t,), linear_logprob(hidden.index_select(0, rows_t), model.output_weight, tgt_t, temperature).float())
        else:
            full = full + 0.0 * hidden.sum()  # a rank without response tokens still takes part in every collective of the backward pass
        return _SumOverRanks.apply(full, cp.comm)


__all__ = ["Qwen3ARStage", "Qwen3ARStep", "Qwen3ARParams", "pack_text_segment", "build_replay_batch"]
