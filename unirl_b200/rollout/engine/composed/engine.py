"""``ComposedRolloutEngine`` — prompt-enhancement flow: an AR child rewrites each prompt ``N`` times, a diffusion child
renders every rewrite ``M`` times.  One request of ``P`` prompts yields two tracks: ``"ar"`` (``P·N`` samples, root) and
``"diffusion"`` (``P·N·M`` samples, child of ``"ar"``).

The children share the GPUs, so the flow is serial with a memory hand-over in between: wake AR / sleep diffusion →
AR generate → extract the rewritten prompt (text after the last ``marker``; a trailing ``</think>`` block is stripped;
an empty extraction falls back to the user's prompt) → sleep AR / wake diffusion → diffusion generate.
Weight-receive calls are demultiplexed by track prefix (``"ar."`` / ``"diffusion."``).
Parity: ``unirl/rollout/engine/composed/engine.py:39-64, 76-106, 154-300, 306-359, 365-506``.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from unirl_b200.distributed.group.dispatch import Dispatch, distributed
from unirl_b200.rollout.engine.base import BaseRolloutEngine
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack


def extract_enhanced_prompt(text: str, user_prompt: str, marker: str = "<prompt>", end_marker: str = "</prompt>") -> str:
    body = text.split("</think>")[-1]
    if marker and marker in body:
        body = body.rsplit(marker, 1)[-1]
    if end_marker and end_marker in body:
        body = body.split(end_marker, 1)[0]
    body = body.strip()
    return body if body else user_prompt


class ComposedRolloutEngine(BaseRolloutEngine):
    _component_name = "composed"

    def __init__(self, *, ar: Any = None, diffusion: Any = None, pe_marker: str = "<prompt>", pe_end_marker: str = "</prompt>",
                 ar_system_instruction: Optional[str] = None, config: Any = None, **_deps: Any) -> None:
        super().__init__()
        if config is not None:  # the configuration-object form: children described by their own engine configurations
            get = (lambda k: config.get(k)) if isinstance(config, dict) else (lambda k: getattr(config, k, None))
            ar = ar if ar is not None else get("ar")
            diffusion = diffusion if diffusion is not None else get("diffusion")
            pe_marker = get("pe_marker") or pe_marker
            ar_system_instruction = get("pe_instruction") or ar_system_instruction
        ar = ar.make_engine() if hasattr(ar, "make_engine") else ar
        diffusion = diffusion.make_engine() if hasattr(diffusion, "make_engine") else diffusion
        if ar is None or diffusion is None:
            raise ValueError("ComposedRolloutEngine needs an autoregressive and a diffusion child engine (objects, or configurations that can build them)")
        self.ar, self.diffusion = ar, diffusion
        self.pe_marker, self.pe_end_marker, self.ar_system_instruction = pe_marker, pe_end_marker, ar_system_instruction

    def _child(self, track_prefix: str) -> Any:
        key = track_prefix.rstrip(".")
        if key not in ("ar", "diffusion"):
            raise ValueError(f"ComposedRolloutEngine: track_prefix must be 'ar.' or 'diffusion.', got {track_prefix!r}")
        return getattr(self, key)

    @distributed(dispatch_mode=Dispatch.DP_SCATTER)
    def generate(self, req: RolloutReq) -> RolloutResp:
        sp = req.sampling_params
        n, m = int(sp.ar.samples_per_prompt), int(sp.diffusion.samples_per_prompt)
        texts = req.primitives.get("text")
        if not isinstance(texts, Texts):
            raise TypeError("ComposedRolloutEngine.generate: req.primitives['text'] must be Texts")
        users = [t.to_str() for t in texts.to_list()]
        # ---- stage 1: AR rewrites ----------------------------------------------------------------------
        self.diffusion.sleep()
        self.ar.wake_up()
        root = req.make_root_track("ar", n)
        chat = dict(req.stage_config.get("chat") or {})
        if self.ar_system_instruction is not None:
            chat.setdefault("system_instruction", self.ar_system_instruction)
        ar_req = RolloutReq(sample_ids=list(root.sample_ids), group_ids=list(root.parent_ids), primitives={"text": texts.repeat_interleave(n)},
                            sampling_params=sp.ar, stage_config={**req.stage_config, "chat": chat})
        ar_track = self.ar.generate(ar_req).tracks["ar"]
        if ar_track.decoded is None:
            raise RuntimeError("ComposedRolloutEngine: the AR child returned no decoded text (enable detokenize)")
        rewrites = [extract_enhanced_prompt(t.to_str(), users[i // n], self.pe_marker, self.pe_end_marker) for i, t in enumerate(ar_track.decoded.to_list())]
        # ---- stage 2: diffusion renders -----------------------------------------------------------------
        self.ar.sleep()
        self.diffusion.wake_up()
        child = ar_track.fork_track("ar", "diffusion", m)
        d = sp.diffusion
        gids = list(child.parent_ids if d.init_same_noise else child.sample_ids)
        diff_req = RolloutReq(sample_ids=list(child.sample_ids), group_ids=list(child.parent_ids),
                              primitives={"text": Texts.from_list([r for r in rewrites for _ in range(m)])}, sampling_params=d, sigmas=req.sigmas,
                              stage_config=dict(req.stage_config), init_noise_group_ids=gids, init_noise_latent_shape=req.init_noise_latent_shape)
        diff_track = self.diffusion.generate(diff_req).tracks["diffusion"]
        diff_track = dataclasses.replace(diff_track, parent_track="ar")
        return RolloutResp(tracks={"ar": ar_track, "diffusion": diff_track})

    # ---- life cycle and weight receive: fan out / demultiplex ---------------------------------------------------
    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def sleep(self) -> None:
        self.ar.sleep()
        self.diffusion.sleep()

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def wake_up(self) -> None:
        return None  # children are woken one at a time inside generate

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def health_check(self) -> bool:
        return bool(self.ar.health_check()) and bool(self.diffusion.health_check())

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def update_weights_from_tensor(self, *, track_prefix: str = "", **kw: Any) -> Any:
        return self._child(track_prefix).update_weights_from_tensor(**kw)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def init_weights_update_group(self, *, track_prefix: str = "", **kw: Any) -> Any:
        return self._child(track_prefix).init_weights_update_group(**kw)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def update_weights_from_distributed(self, *, track_prefix: str = "", **kw: Any) -> Any:
        return self._child(track_prefix).update_weights_from_distributed(**kw)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def destroy_weights_update_group(self, *, track_prefix: str = "", **kw: Any) -> Any:
        return self._child(track_prefix).destroy_weights_update_group(**kw)

    @distributed(dispatch_mode=Dispatch.BROADCAST)
    def set_lora_from_tensors(self, adapter_name: str, lora_tensors: Dict[str, Any], *, track_prefix: str = "", **kw: Any) -> Any:
        return self._child(track_prefix).set_lora_from_tensors(adapter_name, lora_tensors, **kw)


__all__ = ["ComposedRolloutEngine", "extract_enhanced_prompt"]
