"""Slot allocator of the KV pool on top of a prefix-cache manager.

Same behaviour as the reference's ``CacheManager``
(mini_sglang_mlx/scheduler/cache.py:19-90): a free list of slot ids, allocation
that falls back to evicting unlocked cached prefixes, and the hand-over of a
finished request's slots to the prefix cache.  The free list is an int32 tensor
on the pool's device, so ``allocate`` returns ``out_loc`` ready for
``store_kv_cache`` and for the page table.
"""
from __future__ import annotations

import torch

from ..kvcache import BaseCacheHandle, create_cache_manager


class CacheManager:
    def __init__(self, device, num_pages: int, type: str = "radix") -> None:
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self._free_slots = torch.arange(num_pages, dtype=torch.int32, device=self.device)
        self.manager = create_cache_manager(device=self.device, type=type)
        self.num_pages = num_pages

    def _free(self, indices: torch.Tensor) -> None:
        if len(indices) > 0:
            self._free_slots = torch.cat([self._free_slots, indices.to(self.device, torch.int32)])

    def match_req(self, req):
        input_len = req.input_len
        assert input_len > 0, "Input length must be greater than 0."
        # the last prompt token is never served from the cache: its logits are needed
        return self.manager.match_prefix(req.input_ids[: input_len - 1])

    @property
    def available_size(self) -> int:
        return self.manager.size_info.evictable_size + len(self._free_slots)

    def lock(self, handle: BaseCacheHandle) -> None:
        self.manager.lock_handle(handle, unlock=False)

    def unlock(self, handle: BaseCacheHandle) -> None:
        self.manager.lock_handle(handle, unlock=True)

    def allocate(self, needed_len: int) -> torch.Tensor:
        free_len = len(self._free_slots)
        if needed_len > free_len:
            evicted = self.manager.evict(needed_len - free_len)
            self._free_slots = torch.cat([self._free_slots, evicted])
            assert len(self._free_slots) >= needed_len, "Eviction did not free enough space."
        allocated = self._free_slots[:needed_len]
        self._free_slots = self._free_slots[needed_len:]
        return allocated

    def free_and_cache_finished_req(self, old_handle: BaseCacheHandle, input_ids,
                                    indices: torch.Tensor) -> None:
        in_cache_len = self.manager.insert_prefix(input_ids, indices)
        # slots of tokens another request cached in the meantime are duplicates: give them back
        self._free(indices[old_handle.cached_len:in_cache_len])
        self.unlock(old_handle)

    def check_integrity(self) -> None:
        self.manager.check_integrity()
        if len(self._free_slots) + self.manager.size_info.total_size != self.num_pages:
            raise RuntimeError(
                "CacheManager integrity check failed:"
                f" free_slots({len(self._free_slots)}) +"
                f" total_size({self.manager.size_info.total_size}) != num_pages({self.num_pages})")
