"""Vision-language AR stage: the Qwen3 stage plus image features at prefill and 3-axis rotary positions in replay.

Generation hands each sequence's image payload to the paged-KV generator (``extras``); the model merges vision features
into the prompt embeddings during prefill and decode continues with ``cache index + rope_delta`` as the rotary position.
Replay packs ``prompt ⊕ response`` exactly like the text stage; positions of the response tokens continue the prompt's
multimodal positions.  Parity: ``unirl/models/qwen_vl/ar.py:97-213`` (autoregress), ``:215-339`` (replay).
"""

from __future__ import annotations

from typing import Any, List

import torch

from unirl_b200.models.qwen3.ar import Qwen3ARStage, build_replay_batch, pack_text_segment
from unirl_b200.models.qwen3.modeling import AttnMeta
from unirl_b200.models.qwen_vl.conditions import QwenVLARConditions
from unirl_b200.models.types.contracts import unpad_prompts
from unirl_b200.ops.logprob import linear_logprob
from unirl_b200.types.sampling import ARSamplingParams
from unirl_b200.types.segments import TextSegment


class QwenVLARStage(Qwen3ARStage):
    def autoregress(self, conditions: QwenVLARConditions, *, sampling_params: ARSamplingParams, **_kw: Any) -> TextSegment:
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        model = self.model.transformer
        was_training = model.training
        model.eval()
        try:
            out = self.generator.generate(prompts, max_new_tokens=int(sampling_params.max_new_tokens), temperature=float(sampling_params.temperature),
                                          top_k=int(sampling_params.top_k or 0), top_p=float(sampling_params.top_p),
                                          stop_token_ids=self._resolve_stop_ids(sampling_params), extras=conditions.extras())
        finally:
            model.train(was_training)
        return pack_text_segment(out.tokens, out.log_probs, out.finished)

    def replay(self, conditions: QwenVLARConditions, *, segment: TextSegment, temperature: float = 1.0) -> torch.Tensor:
        model = self.model.transformer
        if getattr(model, "cp", None) is not None and model.cp.size > 1:
            raise NotImplementedError("context parallelism is implemented for the text-only replay; vision-language prompts carry image features whose "
                                      "placeholder spans would have to be cut over the ranks")
        device = model.embed_tokens.device
        prompts = unpad_prompts(conditions.prompt.input_ids, conditions.prompt.attention_mask)
        cu = segment.cu_seqlens.tolist()
        responses = [segment.tokens[cu[i] : cu[i + 1]] for i in range(len(cu) - 1)]
        tokens, _pos, cu_dev, max_len, pred_index, targets = build_replay_batch(prompts, responses, device)
        if not targets.numel():
            return torch.zeros(0, dtype=torch.float32, device=device)
        meta = AttnMeta(mode="train", cu_seqlens=cu_dev, max_seqlen=max_len)
        full = [torch.cat([p.to(torch.long).cpu(), r.to(torch.long).cpu()]) for p, r in zip(prompts, responses)]
        extras = conditions.extras() or [None] * len(full)
        model.prepare_multimodal(full, extras, meta, prompt_lens=[len(p) for p in prompts])
        hidden = model(tokens, meta)
        return linear_logprob(hidden.index_select(0, pred_index), model.output_weight, targets, float(temperature))


__all__ = ["QwenVLARStage"]
