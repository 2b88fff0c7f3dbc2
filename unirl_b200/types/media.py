"""``MediaRef`` — a pointer to on-disk / remote media referenced by a dataset row.  Parity: ``unirl/types/media.py``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class MediaRef:
    uri: str
    kind: str = "image"  # image | video | audio
    sha256: Optional[str] = None

    @property
    def is_local(self) -> bool:
        return "://" not in self.uri or self.uri.startswith("file://")

    @property
    def path(self) -> str:
        return self.uri[len("file://"):] if self.uri.startswith("file://") else self.uri


__all__ = ["MediaRef"]
