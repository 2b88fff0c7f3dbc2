"""``Qwen3Pipeline`` — ``RolloutReq`` (texts or pre-tokenised prompts) → one ``"ar"`` track.

Reads ``req.primitives["text"]`` (``Texts``) through the chat template, or — for synthetic-token
workloads — ``req.request_conditions["prompt"]`` (``TextTokenCondition``) verbatim.  Produces
``tracks["ar"]`` with the prompt conditions, the packed ``TextSegment`` and the decoded ``Texts``.
Parity: ``unirl/models/qwen3/pipeline.py:44-211``.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

from unirl_b200.models.qwen3.ar import Qwen3ARParams, Qwen3ARStage
from unirl_b200.models.qwen3.bundle import Qwen3Bundle
from unirl_b200.models.qwen3.chat_template import Qwen3ChatTemplateStage
from unirl_b200.models.qwen3.conditions import Qwen3ARConditions
from unirl_b200.models.qwen3.config import Qwen3PipelineConfig
from unirl_b200.models.types import Pipeline
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack
from unirl_b200.types.sampling import ARSamplingParams, get_ar_params


class Qwen3Pipeline(Pipeline):
    def __init__(self, bundle: Qwen3Bundle, *, enable_thinking: bool = False, system_instruction: Optional[str] = None,
                 autocast_precision: str = "bf16", logprob_precision: str = "fp32", max_prompt_length: int = 2048,
                 generator_kwargs: Optional[dict] = None, detokenize: bool = True):
        super().__init__()
        self.bundle = bundle
        self.chat_template = Qwen3ChatTemplateStage(bundle, system_instruction, max_prompt_length, enable_thinking)
        self.ar = Qwen3ARStage(bundle, autocast_precision, logprob_precision, generator_kwargs)
        self.detokenize = detokenize

    @classmethod
    def from_bundle(cls, bundle: Qwen3Bundle, **kw: Any) -> "Qwen3Pipeline":
        cfg = bundle.config
        kw.setdefault("enable_thinking", cfg.enable_thinking)
        kw.setdefault("system_instruction", cfg.system_instruction)
        kw.setdefault("max_prompt_length", cfg.max_prompt_length)
        return cls(bundle, **kw)

    @classmethod
    def from_config(cls, config: Qwen3PipelineConfig) -> "Qwen3Pipeline":
        return cls.from_bundle(Qwen3Bundle.from_config(config), autocast_precision=config.autocast_precision,
                               logprob_precision=config.logprob_precision)

    def _conditions(self, req: RolloutReq) -> Qwen3ARConditions:
        pre = (req.request_conditions or {}).get("prompt")
        if isinstance(pre, TextTokenCondition):
            return Qwen3ARConditions(prompt=pre)
        texts = req.primitives.get("text")
        if not isinstance(texts, Texts):
            raise TypeError(f"Qwen3Pipeline.generate: req.primitives['text'] must be Texts, got {type(texts).__name__}")
        chat: Dict[str, Any] = dict(req.stage_config.get("chat") or {})
        stage = self.chat_template
        if "system_instruction" in chat:
            stage = Qwen3ChatTemplateStage(self.bundle, chat["system_instruction"], stage.max_prompt_length, stage.enable_thinking)
        return stage.embed(texts)

    def generate(self, req: RolloutReq) -> RolloutResp:
        conds = self._conditions(req)
        ar = get_ar_params(req.sampling_params)
        p = Qwen3ARParams(ar.max_new_tokens, ar.temperature, ar.top_p, ar.top_k) if ar is not None else Qwen3ARParams()
        sp = ARSamplingParams(max_new_tokens=int(p.max_tokens), temperature=float(p.temperature), top_p=float(p.top_p), top_k=int(p.top_k),
                              stop_token_id=getattr(ar, "stop_token_id", None))
        segment = self.ar.autoregress(conds, sampling_params=sp, params=p)
        return RolloutResp(tracks={"ar": RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids), conditions=conds.to_dict(),
                                                      segment=segment, decoded=self._detokenize(segment) if self.detokenize else None)})

    def _detokenize(self, segment: Any) -> Texts:
        if segment.tokens is None or segment.cu_seqlens is None:
            return Texts(texts=[])
        cu = segment.cu_seqlens.tolist()
        tok = self.bundle.tokenizer
        return Texts(texts=[tok.decode(segment.tokens[cu[i] : cu[i + 1]].tolist(), skip_special_tokens=True) for i in range(len(cu) - 1)])


__all__ = ["Qwen3Pipeline"]
