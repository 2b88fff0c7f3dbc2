"""``PEPipeline`` — the composed prompt-enhancement pipeline: an LLM pipeline and a diffusion pipeline behind one
``generate`` (``P`` prompts → ``P·N`` rewrites → ``P·N·M`` images, tracks ``"ar"`` and ``"diffusion"``).

Used by the train-side engine when both models live in the trainer process; the composed rollout engine implements the
same flow over two engine children.  Parity: ``unirl/models/pe/pipeline.py``.
"""

from __future__ import annotations

import dataclasses
from typing import Any

from unirl_b200.models.types import Pipeline
from unirl_b200.rollout.engine.composed.engine import extract_enhanced_prompt
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp


class PEPipeline(Pipeline):
    def __init__(self, diffusion_pipeline: Any, llm_pipeline: Any, pe_marker: str = "<prompt>", pe_end_marker: str = "</prompt>"):
        super().__init__()
        self.diffusion_pipeline, self.llm_pipeline = diffusion_pipeline, llm_pipeline
        self.ar, self.diffusion = llm_pipeline.ar, diffusion_pipeline.diffusion
        self.pe_marker, self.pe_end_marker = pe_marker, pe_end_marker
        self.bundle = diffusion_pipeline.bundle

    def build_schedule_policy(self) -> Any:
        return self.diffusion_pipeline.build_schedule_policy()

    def generate(self, req: RolloutReq) -> RolloutResp:
        sp = req.sampling_params
        n, m = int(sp.ar.samples_per_prompt), int(sp.diffusion.samples_per_prompt)
        texts = req.primitives["text"]
        users = [t.to_str() for t in texts.to_list()]
        root = req.make_root_track("ar", n)
        ar_req = RolloutReq(sample_ids=list(root.sample_ids), group_ids=list(root.parent_ids), primitives={"text": texts.repeat_interleave(n)},
                            sampling_params=sp.ar, stage_config=dict(req.stage_config))
        ar_track = self.llm_pipeline.generate(ar_req).tracks["ar"]
        rewrites = [extract_enhanced_prompt(t.to_str(), users[i // n], self.pe_marker, self.pe_end_marker) for i, t in enumerate(ar_track.decoded.to_list())]
        child = ar_track.fork_track("ar", "diffusion", m)
        d = sp.diffusion
        diff_req = RolloutReq(sample_ids=list(child.sample_ids), group_ids=list(child.parent_ids),
                              primitives={"text": Texts.from_list([r for r in rewrites for _ in range(m)])}, sampling_params=d, sigmas=req.sigmas,
                              stage_config=dict(req.stage_config),
                              init_noise_group_ids=list(child.parent_ids if d.init_same_noise else child.sample_ids),
                              init_noise_latent_shape=req.init_noise_latent_shape)
        diff_track = dataclasses.replace(self.diffusion_pipeline.generate(diff_req).tracks["diffusion"], parent_track="ar")
        return RolloutResp(tracks={"ar": ar_track, "diffusion": diff_track})


__all__ = ["PEPipeline"]
