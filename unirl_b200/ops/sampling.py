"""Token sampler (K12): temperature / top-k / top-p sampling that also returns the log-prob the
trainer will replay — the *full-softmax, temperature-scaled* log-prob recorded before any truncation.

CUDA: one block per row; pass 1 computes the row max and log-sum-exp of ``logits / T``; untruncated
sampling (top_k = 0, top_p = 1, the RL default) draws by Gumbel-max in the same pass with a
counter-based RNG keyed on ``(seed, step, row)``; truncated sampling finds the top-k and top-p thresholds by
radix selection over the row (no sort) and draws among the kept entries with the same random numbers.
No host synchronisation, so the decode loop can live in a CUDA graph either way.
Semantics parity: ``unirl/models/qwen3/ar.py:138-175`` (log-prob before truncation).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                     generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    z = logits.float()
    if temperature <= 0:
        logp = torch.log_softmax(z, -1)
        tok = z.argmax(-1)
        return tok, logp.gather(-1, tok.unsqueeze(-1)).squeeze(-1)
    z = z / temperature
    logp_full = torch.log_softmax(z, -1)
    filt = z
    if top_k and top_k > 0 and top_k < z.shape[-1]:
        kth = torch.topk(filt, top_k, -1).values[..., -1:]
        filt = filt.masked_fill(filt < kth, float("-inf"))
    if top_p < 1.0:
        sv, si = torch.sort(filt, -1, descending=True)
        cum = torch.softmax(sv, -1).cumsum(-1)
        drop = cum - torch.softmax(sv, -1) > top_p
        sv = sv.masked_fill(drop, float("-inf"))
        filt = torch.full_like(filt, float("-inf")).scatter(-1, si, sv)
    tok = torch.multinomial(torch.softmax(filt, -1), 1, generator=generator).squeeze(-1)
    return tok, logp_full.gather(-1, tok.unsqueeze(-1)).squeeze(-1)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, step: int = 0,
           generator: Optional[torch.Generator] = None, out_tokens: Optional[torch.Tensor] = None,
           out_logp: Optional[torch.Tensor] = None, step_tensor: Optional[torch.Tensor] = None, rng_rows: Optional[torch.Tensor] = None,
           rng_steps: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(token [B] int64, logp [B] fp32)``.

    ``step_tensor`` (device int64 scalar) lets a captured graph advance the RNG counter without re-capture.
    ``rng_rows`` / ``rng_steps`` (device int64 ``[B]``, together): key row ``r``'s random stream on ``(rng_rows[r], rng_steps[r])``
    instead of ``(r, step)`` — a generator passes (sequence id, token index), so a sequence draws the same tokens whichever batch
    row it occupies and whenever it was admitted.
    """
    if use_native(logits) and (top_k in (0, None) or top_k >= logits.shape[-1]) and top_p >= 1.0:
        C = require_ext()
        tok, lp = C.sample_full(logits.contiguous(), float(temperature), int(seed), int(step), step_tensor, out_tokens, out_logp, rng_rows, rng_steps)
        count_launch()
        return tok, lp
    if use_native(logits) and temperature > 0 and logits.shape[-1] < (1 << 18) and logits.dtype in (torch.bfloat16, torch.float32):
        C = require_ext()
        tok, lp = C.sample_truncated(logits.contiguous(), float(temperature), int(top_k or 0), float(top_p), int(seed), int(step), step_tensor, out_tokens, out_logp, rng_rows,
                                     rng_steps)
        count_launch()
        return tok, lp
    return sample_reference(logits, temperature, top_k or 0, top_p, generator)


def linear_sample(hidden: torch.Tensor, weight: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
                  step: int = 0, step_tensor: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None,
                  rng_rows: Optional[torch.Tensor] = None, rng_steps: Optional[torch.Tensor] = None):
    """``sample(hidden @ weight.T)`` — on CUDA (bf16, untruncated, T > 0) the vocab projection, the log-sum-exp and the
    Gumbel-max draw run inside ONE tcgen05 GEMM epilogue: the ``[B, vocab]`` logits never reach HBM."""
    fused = (use_native(hidden) and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and temperature > 0
             and (top_k in (0, None) or top_k >= weight.shape[0]) and top_p >= 1.0 and hidden.shape[1] % 8 == 0)
    if fused:
        tok, lp = require_ext().linear_sample(hidden.contiguous(), weight, float(temperature), int(seed), int(step), step_tensor, rng_rows, rng_steps)
        count_launch(2)
        return tok, lp
    logits = torch.nn.functional.linear(hidden, weight)
    return sample(logits, temperature, top_k, top_p, seed=seed, step=step, generator=generator, step_tensor=step_tensor, rng_rows=rng_rows,
                  rng_steps=rng_steps)


__all__ = ["sample", "sample_reference", "linear_sample"]
