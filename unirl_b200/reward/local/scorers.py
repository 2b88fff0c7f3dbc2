"""Model-based image / video scorers as native modules: one vision tower + text tower family covers the preference and
alignment rewards, a vision tower + MLP head covers the aesthetic predictor, rule scorers cover OCR and compositional
checks.

``ClipStyleScorer``     cosine similarity between an image embedding and a prompt embedding, affinely mapped per variant:
                        ``clip`` (raw similarity), ``pickscore`` (logit-scaled), ``hpsv2`` / ``hpsv3`` (x100 human-preference
                        scale), ``image_reward`` (MLP head on the joint feature).
``AestheticScorer``     image embedding → 5-layer MLP → score on the 1–10 scale.
``VideoScorer``         frame-averaged ClipStyleScorer (``videopickscore`` / ``video``) with optional temporal-consistency term.
``OCRScorer``           normalised edit similarity between the text requested in the prompt (between quotes) and the text
                        supplied by an OCR callable (``metadata["ocr_text"]`` when no engine is plugged in).
``GenEvalScorer``       compositional check against ``metadata`` (object counts / colours / positions) given detections in
                        ``metadata["detections"]``.

Published weights: ``model_id`` (or the environment variable ``UNIRL_B200_<VARIANT>_PATH``) names a local directory holding a CLIP-family
checkpoint in the Hugging Face layout (``openai/clip-vit-large-patch14`` for ``clip``, ``yuvalkirstain/PickScore_v1`` with the
``laion/CLIP-ViT-H-14`` processor for ``pickscore``, a converted ViT-H-14 for the HPS variants); the towers are then the published ones, the
images are resized / centre-cropped / normalised on the device as the checkpoint's processor configuration says, and the score follows
the published formula of the variant: ``clip`` = logit_scale · cos / 30, ``pickscore`` = logit_scale · cos / 26, ``hpsv2`` / ``hpsv3`` = cos.
Without ``model_id`` the towers are small random-init stand-ins (native ``TextEncoder`` + a small ViT) with the same score scales, which
keeps recipes runnable without any checkpoint.  Parity: ``unirl/reward/local/{aesthetic,clip,hpsv2,hpsv3,ocr,pickscore,geneval2,
image_reward,videopickscore,video}.py`` (scoring contracts and score scales).
"""

from __future__ import annotations

import re
import time
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from unirl_b200.models.dit.text_encoder import TextEncoder, TextEncoderConfig
from unirl_b200.models.tokenizer import load_tokenizer
from unirl_b200.reward.base import RewardBackend
from unirl_b200.types.reward import RewardRequest, RewardResponse


class _ViT(nn.Module):
    def __init__(self, width: int = 64, layers: int = 2, heads: int = 4, patch: int = 16, image_size: int = 224, out_dim: int = 64):
        super().__init__()
        self.patch, self.image_size = patch, image_size
        self.embed = nn.Conv2d(3, width, patch, patch)
        self.cls = nn.Parameter(torch.zeros(1, 1, width))
        self.pos = nn.Parameter(torch.zeros(1, (image_size // patch) ** 2 + 1, width))
        layer = nn.TransformerEncoderLayer(width, heads, width * 4, 0.0, "gelu", batch_first=True, norm_first=True)
        self.blocks = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
        self.norm, self.proj = nn.LayerNorm(width), nn.Linear(width, out_dim, bias=False)

    def forward(self, px: torch.Tensor) -> torch.Tensor:
        x = F.interpolate(px.float(), size=(self.image_size, self.image_size), mode="bilinear", align_corners=False)
        x = (x - 0.5) / 0.27
        x = self.embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], 1) + self.pos
        return self.proj(self.norm(self.blocks(x)[:, 0]))


class _PublishedClip:
    """A CLIP-family checkpoint in the Hugging Face layout, read from a local directory: towers, tokenizer and preprocessing."""

    def __init__(self, model_path: str, processor_path: Optional[str], device: torch.device):
        import json
        import os

        from transformers import AutoTokenizer, CLIPModel

        if not os.path.isdir(model_path):
            raise FileNotFoundError(f"scorer checkpoint {model_path!r} is not a local directory (checkpoints are never downloaded)")
        self.device = device
        self.model = CLIPModel.from_pretrained(model_path, local_files_only=True).float().eval().requires_grad_(False).to(device)
        proc = processor_path or model_path
        self.tok = AutoTokenizer.from_pretrained(proc, local_files_only=True)
        pre: Dict[str, Any] = {}
        f = os.path.join(proc, "preprocessor_config.json")
        if os.path.exists(f):
            with open(f) as fh:
                pre = json.load(fh)
        self.size = int(self.model.config.vision_config.image_size)
        self.mean = torch.tensor(pre.get("image_mean", [0.48145466, 0.4578275, 0.40821073]), device=device).view(1, 3, 1, 1)
        self.std = torch.tensor(pre.get("image_std", [0.26862954, 0.26130258, 0.27577711]), device=device).view(1, 3, 1, 1)
        self.max_len = int(self.model.config.text_config.max_position_embeddings)

    @staticmethod
    def _features(out: Any) -> torch.Tensor:
        if isinstance(out, torch.Tensor):
            return out
        if getattr(out, "pooler_output", None) is not None:
            return out.pooler_output
        return out[0]

    @torch.no_grad()
    def images(self, px: torch.Tensor) -> torch.Tensor:
        """``[B, 3, H, W]`` in ``[0, 1]`` → unit-norm embeddings (shortest edge to the model's size, bicubic; centre crop; normalise)."""
        x = px.to(self.device).float()
        h, w = x.shape[-2:]
        r = self.size / min(h, w)
        nh, nw = max(self.size, round(h * r)), max(self.size, round(w * r))
        if (nh, nw) != (h, w):
            x = F.interpolate(x, size=(nh, nw), mode="bicubic", antialias=True, align_corners=False).clamp(0, 1)
        top, left = (nh - self.size) // 2, (nw - self.size) // 2
        x = (x[..., top : top + self.size, left : left + self.size] - self.mean) / self.std
        return F.normalize(self._features(self.model.get_image_features(pixel_values=x)), dim=-1)

    @torch.no_grad()
    def texts(self, prompts: List[str]) -> torch.Tensor:
        enc = self.tok(prompts, padding="max_length", truncation=True, max_length=self.max_len, return_tensors="pt")
        enc = {k: v.to(self.device) for k, v in enc.items() if k in ("input_ids", "attention_mask")}
        return F.normalize(self._features(self.model.get_text_features(**enc)), dim=-1)

    @property
    def logit_scale(self) -> torch.Tensor:
        return self.model.logit_scale.exp()


def _pixels_of(request: RewardRequest) -> torch.Tensor:
    gen = request.generated
    for key in ("image", "images"):
        v = gen.get(key)
        if v is not None:
            px = getattr(v, "pixels", v)
            if isinstance(px, torch.Tensor):
                return px
    raise ValueError("image scorer needs generated['image'] (Images or a [B, 3, H, W] tensor in [0, 1])")


def _prompts_of(request: RewardRequest, n: int) -> List[str]:
    t = request.primitives.get("text")
    strs = [x.to_str() if hasattr(x, "to_str") else str(x) for x in (t.to_list() if hasattr(t, "to_list") else (t or []))]
    if not strs:
        return [""] * n
    if len(strs) != n and n % len(strs) == 0:
        strs = [s for s in strs for _ in range(n // len(strs))]
    return strs


class ClipStyleScorer(RewardBackend):
    preferred_input_kind = "image"
    VARIANTS = {"clip": (1.0, 0.0), "pickscore": (100.0, 0.0), "hpsv2": (100.0, 0.0), "hpsv3": (100.0, 0.0), "image_reward": (1.0, 0.0),
                "unified_reward": (5.0, 0.0), "editreward": (1.0, 0.0), "wise": (1.0, 0.0)}

    #: published score of a variant from the cosine similarity and the checkpoint's logit scale
    PUBLISHED = {"clip": lambda cos, ls: ls * cos / 30.0, "pickscore": lambda cos, ls: ls * cos / 26.0, "hpsv2": lambda cos, ls: cos, "hpsv3": lambda cos, ls: cos}

    def __init__(self, variant: str = "clip", width: int = 64, device: Optional[str] = None, seed: int = 0, checkpoint: Optional[str] = None,
                 model_id: Optional[str] = None, processor_id: Optional[str] = None, batch_size: int = 8, **_kw: Any):
        import os

        if variant not in self.VARIANTS:
            raise ValueError(f"unknown scorer variant {variant!r}; known: {sorted(self.VARIANTS)}")
        self.variant, (self.scale, self.bias) = variant, self.VARIANTS[variant]
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.batch_size = max(1, int(batch_size))
        model_id = model_id or os.environ.get(f"UNIRL_B200_{variant.upper()}_PATH")
        self.published = _PublishedClip(model_id, processor_id, self.device) if model_id else None
        if self.published is not None:
            self.vision = self.text = self.tok = self.head = None
            return
        torch.manual_seed(seed)
        self.vision = _ViT(width, out_dim=width).to(self.device).eval().requires_grad_(False)
        self.text = TextEncoder(TextEncoderConfig.tiny("clip", hidden=width, vocab=4096, max_length=77), dtype=torch.float32, device=self.device).init_weights(seed + 1)
        self.tok = load_tokenizer(None, 4096, True)
        self.head = nn.Sequential(nn.Linear(2 * width, width), nn.GELU(), nn.Linear(width, 1)).to(self.device).eval().requires_grad_(False) if variant == "image_reward" else None
        if checkpoint:
            sd = torch.load(checkpoint, map_location=self.device)
            self.vision.load_state_dict(sd["vision"])
            self.text.load_state_dict(sd["text"])

    def get_model_name(self) -> str:
        return self.variant

    @torch.no_grad()
    def _embed_text(self, prompts: List[str]) -> torch.Tensor:
        c = self.text.cfg
        rows = [([int(i) % c.vocab_size for i in self.tok.encode(p)][: c.max_length - 1] + [c.eos_token_id]) for p in prompts]
        ids = torch.full((len(rows), c.max_length), c.eos_token_id, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : len(r)] = torch.tensor(r)
        return self.text(ids.to(self.device))[1]

    @torch.no_grad()
    def score(self, pixels: torch.Tensor, prompts: List[str]) -> torch.Tensor:
        if self.published is not None:
            out = []
            for i in range(0, pixels.shape[0], self.batch_size):
                cos = (self.published.images(pixels[i : i + self.batch_size]) * self.published.texts(prompts[i : i + self.batch_size])).sum(-1)
                fn = self.PUBLISHED.get(self.variant)
                out.append(fn(cos, self.published.logit_scale) if fn is not None else cos * self.scale + self.bias)
            return torch.cat(out)
        img = self.vision(pixels.to(self.device))
        txt = self._embed_text(prompts)
        if self.head is not None:
            return self.head(torch.cat([img, txt], -1)).squeeze(-1)
        return F.cosine_similarity(img, txt, dim=-1) * self.scale + self.bias

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        px = _pixels_of(request)
        s = self.score(px, _prompts_of(request, px.shape[0]))
        return RewardResponse.ok(s.float().cpu().tolist(), {self.variant: s.float().cpu().tolist()}, time.perf_counter() - t0)

    def offload(self) -> None:
        if self.published is not None:
            self.published.model.to("cpu")
        else:
            self.vision.to("cpu"), self.text.to("cpu")

    def onload(self) -> None:
        if self.published is not None:
            self.published.model.to(self.device)
        else:
            self.vision.to(self.device), self.text.to(self.device)


class AestheticScorer(RewardBackend):
    preferred_input_kind = "image"

    def __init__(self, width: int = 64, device: Optional[str] = None, seed: int = 0, **_kw: Any):
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        torch.manual_seed(seed)
        self.vision = _ViT(width, out_dim=width).to(self.device).eval().requires_grad_(False)
        dims = [width, 1024, 128, 64, 16, 1]
        self.mlp = nn.Sequential(*[m for a, b in zip(dims[:-1], dims[1:]) for m in (nn.Linear(a, b),)]).to(self.device).eval().requires_grad_(False)

    @torch.no_grad()
    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        emb = F.normalize(self.vision(_pixels_of(request).to(self.device)), dim=-1)
        s = (5.5 + 4.5 * torch.tanh(self.mlp(emb).squeeze(-1))).cpu().tolist()  # 1..10 scale
        return RewardResponse.ok(s, {"aesthetic": s}, time.perf_counter() - t0)


class VideoScorer(RewardBackend):
    preferred_input_kind = "video"

    def __init__(self, variant: str = "pickscore", temporal_weight: float = 0.0, **kw: Any):
        self.frame_scorer = ClipStyleScorer(variant=variant, **kw)
        self.temporal_weight = float(temporal_weight)

    @torch.no_grad()
    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        vids = request.generated.get("video")
        clips = vids.to_list() if hasattr(vids, "to_list") else vids
        prompts = _prompts_of(request, len(clips))
        out = []
        for clip, p in zip(clips, prompts):
            fr = getattr(clip, "frames", clip)
            s = self.frame_scorer.score(fr, [p] * fr.shape[0]).mean()
            if self.temporal_weight and fr.shape[0] > 1:
                s = s - self.temporal_weight * (fr[1:].float() - fr[:-1].float()).abs().mean()
            out.append(float(s))
        return RewardResponse.ok(out, {"video": out}, time.perf_counter() - t0)


def _edit_similarity(a: str, b: str) -> float:
    a, b = a.lower().strip(), b.lower().strip()
    if not a and not b:
        return 1.0
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return 1.0 - prev[-1] / max(len(a), len(b), 1)


class OCRScorer(RewardBackend):
    preferred_input_kind = "image"

    def __init__(self, ocr_fn: Optional[Callable[[torch.Tensor], str]] = None, **_kw: Any):
        self.ocr_fn = ocr_fn

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        px = _pixels_of(request)
        prompts = _prompts_of(request, px.shape[0])
        meta = request.metadata or [None] * px.shape[0]
        if len(meta) != px.shape[0] and px.shape[0] % max(1, len(meta)) == 0:
            meta = [m for m in meta for _ in range(px.shape[0] // len(meta))]
        out = []
        for i, p in enumerate(prompts):
            want = " ".join(re.findall(r'"([^"]+)"', p)) or (meta[i] or {}).get("target_text", "")
            got = self.ocr_fn(px[i]) if self.ocr_fn is not None else str((meta[i] or {}).get("ocr_text", ""))
            out.append(_edit_similarity(want, got))
        return RewardResponse.ok(out, {"ocr": out}, time.perf_counter() - t0)


class GenEvalScorer(RewardBackend):
    """``metadata[i]["include"] = [{"class": "dog", "count": 2, "color": "red"}, …]`` checked against
    ``metadata[i]["detections"] = [{"class": "dog", "color": "red"}, …]``; reward = fraction of satisfied requirements."""

    preferred_input_kind = "image"

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        meta = request.metadata or []
        n = request.batch_size or len(meta)
        if meta and len(meta) != n and n % len(meta) == 0:
            meta = [m for m in meta for _ in range(n // len(meta))]
        out = []
        for m in (meta or [None] * n):
            req, det = (m or {}).get("include", []), (m or {}).get("detections", [])
            if not req:
                out.append(0.0)
                continue
            ok = 0
            for r in req:
                hits = [d for d in det if d.get("class") == r.get("class") and (r.get("color") is None or d.get("color") == r.get("color"))]
                ok += int(len(hits) >= int(r.get("count", 1)))
            out.append(ok / len(req))
        return RewardResponse.ok(out, {"geneval": out}, time.perf_counter() - t0)


SCORERS: Dict[str, Callable[..., RewardBackend]] = {
    "clip": lambda **k: ClipStyleScorer("clip", **k), "pickscore": lambda **k: ClipStyleScorer("pickscore", **k), "hpsv2": lambda **k: ClipStyleScorer("hpsv2", **k),
    "hpsv3": lambda **k: ClipStyleScorer("hpsv3", **k), "image_reward": lambda **k: ClipStyleScorer("image_reward", **k),
    "imagereward": lambda **k: ClipStyleScorer("image_reward", **k), "unified_reward": lambda **k: ClipStyleScorer("unified_reward", **k),
    "editreward": lambda **k: ClipStyleScorer("editreward", **k), "wise": lambda **k: ClipStyleScorer("wise", **k), "aesthetic": lambda **k: AestheticScorer(**k),
    "ocr": lambda **k: OCRScorer(**k), "geneval": lambda **k: GenEvalScorer(), "geneval2": lambda **k: GenEvalScorer(),
    "videopickscore": lambda **k: VideoScorer("pickscore", **k), "video": lambda **k: VideoScorer("clip", temporal_weight=0.1, **k),
    "videoalign": lambda **k: VideoScorer("clip", **k),
}


def build_scorer(name: str, **kw: Any) -> RewardBackend:
    if name not in SCORERS:
        raise KeyError(f"unknown scorer {name!r}; known: {sorted(SCORERS)}")
    return SCORERS[name](**kw)


__all__ = ["ClipStyleScorer", "AestheticScorer", "VideoScorer", "OCRScorer", "GenEvalScorer", "SCORERS", "build_scorer"]
