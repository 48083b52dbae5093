"""Cache manager that caches nothing (reference: mini_sglang_mlx/kvcache/naive_manager.py:14-44)."""
from __future__ import annotations

from typing import Tuple

import torch

from .base import BaseCacheHandle, SizeInfo


class NaiveCacheHandle(BaseCacheHandle):
    pass


class NaiveCacheManager:
    def __init__(self, device=None) -> None:
        self.empty_tensor = torch.zeros(0, dtype=torch.int32, device=device or "cpu")

    def match_prefix(self, input_ids) -> Tuple[NaiveCacheHandle, torch.Tensor]:
        return NaiveCacheHandle(0), self.empty_tensor

    def lock_handle(self, handle: BaseCacheHandle, unlock: bool = False) -> None:
        pass

    def insert_prefix(self, input_ids, indices: torch.Tensor) -> int:
        assert len(indices) == len(input_ids)
        return len(indices)

    def evict(self, size: int) -> torch.Tensor:
        if size == 0:
            return self.empty_tensor
        raise NotImplementedError("NaiveCacheManager does not support eviction.")

    def reset(self) -> None:
        pass

    @property
    def size_info(self) -> SizeInfo:
        return SizeInfo(0, 0)

    def check_integrity(self) -> None:
        pass
