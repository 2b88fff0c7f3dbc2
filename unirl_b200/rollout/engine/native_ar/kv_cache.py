"""Paged KV cache and its block allocator.

Layout per layer: ``[num_pages, Hkv, page_size, D]`` (K and V separate) so that one (page, head)
block is a contiguous slab the decode kernel can stream with bulk copies.  The allocator is a
free-list over page ids; the native build swaps in the C++ allocator (``_C.BlockAllocator``) with
the same interface.  ``release()`` drops the tensors so a colocated trainer can use the HBM
(the ``sleep``/``wake_up`` contract of the rollout engines, ``unirl/rollout/engine/base.py:45-192``).
"""

from __future__ import annotations

from typing import List, Optional

import torch


class BlockAllocator:
    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n > len(self._free):
            raise MemoryError(f"KV cache exhausted: need {n} pages, {len(self._free)} free of {self.num_pages}")
        got = self._free[-n:][::-1] if n else []
        del self._free[len(self._free) - n :]
        return got

    def free(self, pages: List[int]) -> None:
        self._free.extend(reversed(pages))

    def reset(self) -> None:
        self._free = list(range(self.num_pages - 1, -1, -1))


def make_allocator(num_pages: int):
    from unirl_b200.ops._ext import ext

    C = ext()
    if C is not None and hasattr(C, "BlockAllocator"):
        return C.BlockAllocator(int(num_pages))
    return BlockAllocator(num_pages)


class PagedKVCache:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, page_size: int, num_pages: int, dtype: torch.dtype, device):
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.page_size, self.num_pages, self.dtype, self.device = page_size, int(num_pages), dtype, torch.device(device)
        self.k: Optional[List[torch.Tensor]] = None
        self.v: Optional[List[torch.Tensor]] = None
        self.allocator = make_allocator(self.num_pages)
        self.allocate()

    @staticmethod
    def bytes_per_token(num_layers: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> int:
        return 2 * num_layers * num_kv_heads * head_dim * torch.empty(0, dtype=dtype).element_size()

    def allocate(self) -> None:
        if self.k is not None:
            return
        shape = (self.num_pages, self.num_kv_heads, self.page_size, self.head_dim)
        # one slab per layer: a single 2*L*pages allocation would need a >100 GB contiguous range
        self.k = [torch.zeros(shape, dtype=self.dtype, device=self.device) for _ in range(self.num_layers)]
        self.v = [torch.zeros(shape, dtype=self.dtype, device=self.device) for _ in range(self.num_layers)]

    def release(self) -> None:
        self.k = self.v = None
        self.allocator.reset()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    @property
    def is_allocated(self) -> bool:
        return self.k is not None

    def nbytes(self) -> int:
        return 0 if self.k is None else 2 * self.num_layers * self.k[0].numel() * self.k[0].element_size()


__all__ = ["BlockAllocator", "PagedKVCache", "make_allocator"]
