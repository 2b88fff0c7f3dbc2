"""Raw (pre-encoder) inputs and decoded outputs: single items and their batched containers.

``Texts`` is a list of strings; ``Images`` a ``[B, C, H, W]`` tensor; ``Videos`` / ``Audios`` pack
ragged frame / sample counts along dim 0.  Parity: ``unirl/types/primitives.py:64-295``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, packed_field, shared_field


@dataclass
class Text:
    text: str = ""

    @classmethod
    def from_str(cls, s: str) -> "Text":
        return cls(text=str(s))

    def to_str(self) -> str:
        return self.text


@dataclass
class Embedding:
    values: Optional[torch.Tensor] = None


@dataclass
class Image:
    pixels: Optional[torch.Tensor] = None  # [C, H, W] in [0, 1]

    def to_pil(self):
        from PIL import Image as PILImage

        arr = (self.pixels.detach().float().clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
        return PILImage.fromarray(arr.squeeze(-1) if arr.shape[-1] == 1 else arr)


@dataclass
class Video:
    frames: Optional[torch.Tensor] = None  # [F, C, H, W]
    fps: float = 16.0

    def to_pils(self):
        return [Image(f).to_pil() for f in self.frames]


@dataclass
class Audio:
    waveform: Optional[torch.Tensor] = None  # [T, channels]
    sample_rate: int = 16000


@dataclass
class TextAndImage:
    text: Text = None
    image: Image = None


@dataclass
class TextAndVideo:
    text: Text = None
    video: Video = None


@dataclass
class Texts(Batch):
    texts: List[str] = concat_field(default_factory=list)

    @classmethod
    def from_list(cls, items: List[Any]) -> "Texts":
        return cls(texts=[i.to_str() if isinstance(i, Text) else str(i) for i in items])

    def to_list(self) -> List[Text]:
        return [Text(t) for t in self.texts]

    def __len__(self) -> int:
        return len(self.texts)


@dataclass
class Images(Batch):
    pixels: Optional[torch.Tensor] = concat_field(default=None)  # [B, C, H, W]

    @classmethod
    def from_list(cls, items: List[Image]) -> "Images":
        if not items:
            return cls(pixels=None)
        shapes = {tuple(i.pixels.shape) for i in items}
        if len(shapes) > 1:
            raise ValueError(f"Images.from_list needs same-shaped images, got {sorted(shapes)}")
        return cls(pixels=torch.stack([i.pixels for i in items]))

    def to_list(self) -> List[Image]:
        return [] if self.pixels is None else [Image(p) for p in self.pixels]

    def __len__(self) -> int:
        return 0 if self.pixels is None else int(self.pixels.shape[0])


@dataclass
class Videos(Batch):
    frames: Optional[torch.Tensor] = packed_field(default=None)  # [sum F_i, C, H, W]
    fps: float = shared_field(default=16.0)

    @property
    def cu_frames(self) -> Optional[torch.Tensor]:
        return self.cu_seqlens

    @classmethod
    def from_list(cls, items: List[Video]) -> "Videos":
        return cls.pack(frames=[v.frames for v in items], fps=items[0].fps if items else 16.0)

    def to_list(self) -> List[Video]:
        cu = self.cu_seqlens.tolist()
        return [Video(self.frames[cu[i] : cu[i + 1]], self.fps) for i in range(len(cu) - 1)]

    def __len__(self) -> int:
        return self.batch_size


@dataclass
class Audios(Batch):
    waveform: Optional[torch.Tensor] = packed_field(default=None)
    sample_rate: int = shared_field(default=16000)

    @property
    def cu_samples(self) -> Optional[torch.Tensor]:
        return self.cu_seqlens

    @classmethod
    def from_list(cls, items: List[Audio]) -> "Audios":
        return cls.pack(waveform=[a.waveform for a in items], sample_rate=items[0].sample_rate if items else 16000)

    def to_list(self) -> List[Audio]:
        cu = self.cu_seqlens.tolist()
        return [Audio(self.waveform[cu[i] : cu[i + 1]], self.sample_rate) for i in range(len(cu) - 1)]

    def __len__(self) -> int:
        return self.batch_size


__all__ = ["Text", "Embedding", "Image", "Video", "Audio", "TextAndImage", "TextAndVideo", "Texts", "Images", "Videos", "Audios"]
