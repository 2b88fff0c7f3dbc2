"""Stages of the unified model: text generation / replay and flow-matching denoising on the SAME transformer.

``UnifiedARStage``         greedy-free sampling loop with a dense KV cache (left-aligned prompts, per-row finished latch) and
                           teacher-forced replay through the fused ``linear → log-softmax → gather`` op.
``UnifiedDiffusionStage``  the DiT diffusion stage with the velocity coming from ``forward_image`` conditioned on prompt
                           token ids (not on encoder embeddings); classifier-free guidance uses an empty prompt.
Parity: ``unirl/models/hunyuan_image3/{ar,diffusion}.py``, ``unirl/models/bagel/diffusion.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.models.dit.diffusion import DiTDiffusionParams, DiTDiffusionStage
from unirl_b200.models.qwen3.ar import pack_text_segment
from unirl_b200.models.types.contracts import unpad_prompts
from unirl_b200.ops.logprob import linear_logprob
from unirl_b200.ops.sampling import sample_reference
from unirl_b200.types.conditions import Condition, ImageLatentCondition, TextTokenCondition
from unirl_b200.types.sampling import ARSamplingParams
from unirl_b200.types.segments import TextSegment


@dataclass
class UnifiedConditions(Batch):
    """Prompt token ids (both modes), optional negative prompt (image mode CFG), optional source-image latents."""

    prompt: Optional[TextTokenCondition] = concat_field(default=None)
    negative_prompt: Optional[TextTokenCondition] = concat_field(default=None)
    image: Optional[ImageLatentCondition] = concat_field(default=None)

    @classmethod
    def from_dict(cls, d: Dict[str, Condition]) -> "UnifiedConditions":
        if not isinstance(d.get("prompt"), TextTokenCondition):
            raise TypeError("UnifiedConditions: d['prompt'] must be a TextTokenCondition")
        return cls(prompt=d["prompt"], negative_prompt=d.get("negative_prompt"), image=d.get("image"))

    def to_dict(self) -> Dict[str, Condition]:
        out: Dict[str, Condition] = {"prompt": self.prompt}
        if self.negative_prompt is not None:
            out["negative_prompt"] = self.negative_prompt
        if self.image is not None:
            out["image"] = self.image
        return out


class UnifiedARStage:
    def __init__(self, bundle: Any):
        self.model = bundle

    def trainable_module(self) -> torch.nn.Module:
        return self.model.transformer

    @torch.no_grad()
    def autoregress(self, conditions: UnifiedConditions, *, sampling_params: ARSamplingParams, **_kw: Any) -> TextSegment:
        m = self.model.transformer
        dev = m.embed_tokens.device
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        b, max_new = len(prompts), int(sampling_params.max_new_tokens)
        stop = {int(m.cfg.eos_token_id)} | ({int(sampling_params.stop_token_id)} if sampling_params.stop_token_id is not None else set())
        toks: List[List[int]] = [[] for _ in range(b)]
        lps: List[List[float]] = [[] for _ in range(b)]
        finished = torch.zeros(b, dtype=torch.bool)
        gen = torch.Generator().manual_seed(int(getattr(self.model.config, "init_seed", 0)) + 17)
        was = m.training
        m.eval()
        try:
            for i, p in enumerate(prompts):  # one sequence at a time keeps the dense cache free of padding
                caches = [{} for _ in m.layers]
                ids = p.to(dev).long()[None]
                h = m.forward_text(ids, torch.ones_like(ids), caches)
                n = ids.shape[1]
                for _ in range(max_new):
                    logits = torch.nn.functional.linear(h[:, -1].float(), m.output_weight.float()).cpu()
                    t, lp = sample_reference(logits, float(sampling_params.temperature), int(sampling_params.top_k or 0), float(sampling_params.top_p), gen)
                    toks[i].append(int(t))
                    lps[i].append(float(lp))
                    if int(t) in stop:
                        finished[i] = True
                        break
                    nxt = torch.tensor([[int(t)]], device=dev)
                    h = m.forward_text(nxt, torch.ones_like(nxt), caches, positions=torch.tensor([[n]], device=dev), key_mask=torch.ones(1, n + 1, device=dev))
                    n += 1
        finally:
            m.train(was)
        return pack_text_segment([torch.tensor(t) for t in toks], [torch.tensor(l) for l in lps], finished)

    def replay(self, conditions: UnifiedConditions, *, segment: TextSegment, temperature: float = 1.0) -> torch.Tensor:
        m = self.model.transformer
        dev = m.embed_tokens.device
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        cu = segment.cu_seqlens.tolist()
        hidden, targets = [], []
        rows = [torch.cat([p.long(), segment.tokens[cu[i] : cu[i + 1]].long()]) for i, p in enumerate(prompts)]
        width = max(int(r.numel()) for r in rows)
        ids = torch.full((len(rows), width), int(m.cfg.pad_token_id), dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : r.numel()], mask[i, : r.numel()] = r, 1
        h = m.forward_text(ids.to(dev), mask.to(dev))
        for i, p in enumerate(prompts):
            n_p, n_r = int(p.numel()), cu[i + 1] - cu[i]
            if n_r:
                hidden.append(h[i, n_p - 1 : n_p + n_r - 1])
                targets.append(segment.tokens[cu[i] : cu[i + 1]].long())
        if not hidden:
            return torch.zeros(0, dtype=torch.float32, device=dev)
        return linear_logprob(torch.cat(hidden), m.output_weight, torch.cat(targets).to(dev), float(temperature))


class UnifiedDiffusionStage(DiTDiffusionStage):
    def __init__(self, bundle: Any, default_strategy: str = "flow", autocast_precision: str = "bf16"):
        super().__init__(bundle, default_strategy, autocast_precision)

    def _branches(self, x: torch.Tensor, sigma: torch.Tensor, cond: UnifiedConditions, p: DiTDiffusionParams):
        """``(v_cond, v_uncond | None)`` of one transformer evaluation in image mode (the base class combines them, or hands both to the
        SDE-step kernel)."""
        m = self.bundle.transformer
        t = sigma.to(x.device).float().reshape(-1).expand(x.shape[0]) * 1000.0
        ids, mask = cond.prompt.input_ids.to(x.device), cond.prompt.attention_mask.to(x.device)
        if not (p.guidance_scale > 1.0 and cond.negative_prompt is not None):
            return m.forward_image(ids, mask, x, t).float(), None
        nids, nmask = cond.negative_prompt.input_ids.to(x.device), cond.negative_prompt.attention_mask.to(x.device)
        width = max(ids.shape[1], nids.shape[1])
        pad = lambda a, v: torch.nn.functional.pad(a, (0, width - a.shape[1]), value=v)  # noqa: E731
        v = m.forward_image(torch.cat([pad(nids, int(m.cfg.pad_token_id)), pad(ids, int(m.cfg.pad_token_id))]), torch.cat([pad(nmask, 0), pad(mask, 0)]),
                            torch.cat([x, x]), torch.cat([t, t])).float()
        vu, vc = v.chunk(2)
        return vc, vu


__all__ = ["UnifiedConditions", "UnifiedARStage", "UnifiedDiffusionStage"]
