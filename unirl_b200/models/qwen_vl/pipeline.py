"""``QwenVLPipeline`` — ``RolloutReq`` with ``Texts`` (+ optional ``Images``) → one ``"ar"`` track.

Every image becomes ``<|vision_start|> <|image_pad|>·(t·h·w/4) <|vision_end|>`` in front of the question; patches are
produced by :mod:`unirl_b200.models.qwen_vl.processor`.  Parity: ``unirl/models/qwen_vl/pipeline.py:19-125``,
``unirl/models/qwen_vl/chat_template.py``.
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch

from unirl_b200.models.qwen_vl.ar import QwenVLARStage
from unirl_b200.models.qwen_vl.bundle import QwenVLBundle
from unirl_b200.models.qwen_vl.conditions import QwenVLARConditions
from unirl_b200.models.qwen_vl.config import QwenVLPipelineConfig
from unirl_b200.models.qwen_vl.processor import preprocess_image
from unirl_b200.models.types import Pipeline
from unirl_b200.types.conditions import TextTokenCondition
from unirl_b200.types.primitives import Images, Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack
from unirl_b200.types.sampling import ARSamplingParams, get_ar_params


class QwenVLPipeline(Pipeline):
    conditions_cls = QwenVLARConditions

    def __init__(self, bundle: QwenVLBundle, *, detokenize: bool = True, generator_kwargs: Optional[dict] = None, max_prompt_length: Optional[int] = None,
                 autocast_precision: Optional[str] = None, logprob_precision: Optional[str] = None, **_ignored: Any):
        """The precision and prompt-length options override the bundle's configuration (recipes may give them on the pipeline)."""
        super().__init__()
        self.bundle = bundle
        for name, value in (("max_prompt_length", max_prompt_length), ("autocast_precision", autocast_precision), ("logprob_precision", logprob_precision)):
            if value is not None and hasattr(bundle.config, name):
                setattr(bundle.config, name, value)
        self.ar = QwenVLARStage(bundle, bundle.config.autocast_precision, bundle.config.logprob_precision, generator_kwargs)
        self.detokenize = detokenize

    @classmethod
    def from_bundle(cls, bundle: QwenVLBundle, **kw: Any) -> "QwenVLPipeline":
        return cls(bundle, **kw)

    @classmethod
    def from_config(cls, config: QwenVLPipelineConfig) -> "QwenVLPipeline":
        return cls(QwenVLBundle.from_config(config))

    def _conditions(self, req: RolloutReq) -> QwenVLARConditions:
        pre = req.request_conditions or {}
        if isinstance(pre.get("prompt"), TextTokenCondition):
            return QwenVLARConditions.from_dict(pre)
        texts, images = req.primitives.get("text"), req.primitives.get("image")
        if not isinstance(texts, Texts):
            raise TypeError("QwenVLPipeline.generate: req.primitives['text'] must be Texts")
        cfg, tok, bc = self.bundle.model_config, self.bundle.tokenizer, self.bundle.config
        rows: List[List[int]] = []
        pvs: List[Any] = []
        grids: List[Any] = []
        for i, t in enumerate(texts.to_list()):
            ids: List[int] = []
            pv = g = None
            if isinstance(images, Images) and images.pixels is not None:
                pv, grid = preprocess_image(images.pixels[i], cfg.vision, bc.min_pixels, bc.max_pixels)
                n = grid[0] * grid[1] * grid[2] // cfg.vision.spatial_merge_size**2
                ids += [cfg.vision_start_token_id] + [cfg.image_token_id] * n
                g = torch.tensor([grid])
            reserved = {cfg.image_token_id, cfg.video_token_id, cfg.vision_start_token_id}
            ids += [int(x) % cfg.vocab_size if int(x) % cfg.vocab_size not in reserved else 10 for x in tok.encode(t.to_str())][: bc.max_prompt_length]
            rows.append(ids)
            pvs.append(pv)
            grids.append(g)
        width = max(len(r) for r in rows)
        input_ids = torch.full((len(rows), width), int(cfg.pad_token_id), dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            input_ids[i, : len(r)] = torch.tensor(r)
            mask[i, : len(r)] = 1
        has_img = any(p is not None for p in pvs)
        return QwenVLARConditions(prompt=TextTokenCondition(input_ids=input_ids, attention_mask=mask), pixel_values=pvs if has_img else None,
                                  image_grid_thw=grids if has_img else None)

    def generate(self, req: RolloutReq) -> RolloutResp:
        conds = self._conditions(req)
        ar = get_ar_params(req.sampling_params) or ARSamplingParams()
        seg = self.ar.autoregress(conds, sampling_params=ar)
        decoded = None
        if self.detokenize and seg.tokens is not None:
            cu = seg.cu_seqlens.tolist()
            decoded = Texts(texts=[self.bundle.tokenizer.decode(seg.tokens[cu[i] : cu[i + 1]].tolist(), skip_special_tokens=True) for i in range(len(cu) - 1)])
        return RolloutResp(tracks={"ar": RolloutTrack(sample_ids=list(req.sample_ids), parent_ids=list(req.group_ids), conditions=conds.to_dict(),
                                                      segment=seg, decoded=decoded)})


__all__ = ["QwenVLPipeline"]
