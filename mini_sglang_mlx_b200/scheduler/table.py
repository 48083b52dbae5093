"""Rows of the page table handed out to running requests
(reference: mini_sglang_mlx/scheduler/table.py:4-21)."""
from __future__ import annotations

import torch


class TableManager:
    def __init__(self, max_running_reqs: int, page_table: torch.Tensor) -> None:
        self._max_running_reqs = max_running_reqs
        self._free_slots = list(range(max_running_reqs))
        self.page_table = page_table
        # token ids of every table row; the dummy padding request reads it, so it starts as zeros
        self.token_pool = torch.zeros_like(page_table)

    @property
    def available_size(self) -> int:
        return len(self._free_slots)

    def allocate(self) -> int:
        return self._free_slots.pop()

    def free(self, slot: int) -> None:
        self._free_slots.append(slot)
