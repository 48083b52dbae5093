"""The two scheduler-side records the attention backend reads.

Field names and meaning follow the reference's ``Req`` and ``Batch``
(mini_sglang_mlx/core.py:35-147); only the fields the attention path touches
are kept, so a scheduler written against the reference can hand its own
objects over unchanged (duck typing).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch


class BatchPhase(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    TARGET_VERIFY = "target_verify"


@dataclass(eq=False)
class Req:
    """A running request: row ``table_idx`` of the page table holds its slot
    ids; ``cached_len`` tokens already have K/V in the pool, ``device_len``
    tokens will have after this step."""
    table_idx: int
    cached_len: int
    device_len: int

    def __post_init__(self) -> None:
        assert 0 <= self.cached_len < self.device_len

    @property
    def extend_len(self) -> int:
        return self.device_len - self.cached_len

    def complete_one(self) -> None:
        self.cached_len = self.device_len
        self.device_len += 1

    def complete_many(self, n: int) -> None:
        self.cached_len += n
        self.device_len = self.cached_len + 1


@dataclass
class Batch:
    reqs: List[Req]
    phase: BatchPhase
    out_loc: Optional[torch.Tensor] = None          # (N,) int32 slots the new K/V rows go to
    padded_reqs: List[Req] = field(default_factory=list)
    attn_metadata: Any = None

    def __post_init__(self) -> None:
        if not self.padded_reqs:
            self.padded_reqs = list(self.reqs)

    @property
    def is_prefill(self) -> bool:
        return self.phase == BatchPhase.PREFILL

    @property
    def is_decode(self) -> bool:
        return self.phase == BatchPhase.DECODE

    @property
    def size(self) -> int:
        return len(self.reqs)
