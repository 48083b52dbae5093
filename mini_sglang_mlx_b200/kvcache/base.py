"""Interfaces of the prefix-cache managers: field and method names follow the
reference's ``BaseCacheHandle`` / ``SizeInfo`` / ``BaseCacheManager``
(mini_sglang_mlx/kvcache/base.py:36-121)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple


@dataclass(frozen=True)
class BaseCacheHandle:
    cached_len: int


class SizeInfo(NamedTuple):
    evictable_size: int
    protected_size: int

    @property
    def total_size(self) -> int:
        return self.evictable_size + self.protected_size
