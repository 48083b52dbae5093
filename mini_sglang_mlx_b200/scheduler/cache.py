"""Slot allocator of the KV pool on top of a prefix-cache manager.

Same behaviour as the reference's ``CacheManager``
(mini_sglang_mlx/scheduler/cache.py:19-90): a free list, allocation that falls
back to evicting unlocked cached prefixes, and the hand-over of a finished
request's slots to the prefix cache.  ``allocate`` returns per-token slot ids
(int32, on the pool's device) ready for ``store_kv_cache`` and for the page
table.

``page_size`` > 1 (the reference allocates single tokens,
scheduler/cache.py:45-57) makes the allocation page-granular, which is what the
page-granular attention entries need: the free list holds PAGE ids, a request's
tokens fill its last page before a new page is taken (token t of a request sits
in slot ``page(t // page_size) * page_size + t % page_size``), the prefix cache
takes over whole pages only, and the partial last page of a finished request goes
back to the free list.  The free list is a host-side queue served in the reference's
order (allocate from the front, free to the back), so the slot ids a run produces are
the reference's; nothing on the device is resized per call.
"""
from __future__ import annotations

from collections import deque
from typing import List, Optional

import torch

from ..kvcache import BaseCacheHandle, create_cache_manager


class CacheManager:
    def __init__(self, device, num_pages: int, type: str = "radix", page_size: int = 1) -> None:
        assert page_size >= 1
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.page_size = page_size
        self._free_pages = deque(range(num_pages))
        self.manager = create_cache_manager(device=self.device, type=type, page_size=page_size)
        self.num_pages = num_pages

    # ------------------------------------------------------------------ free list
    def _pages_of(self, slots: torch.Tensor) -> List[int]:
        """Pages of a run of per-token slots that starts on a page boundary (a trailing partial
        page counts)."""
        if len(slots) == 0:
            return []
        first = slots[:: self.page_size]
        if self.page_size > 1:
            first = first // self.page_size
        return first.tolist()

    def _free(self, indices: torch.Tensor) -> None:
        self._free_pages.extend(self._pages_of(indices))

    @property
    def _free_slots(self) -> torch.Tensor:
        """The free pages as a tensor (kept for callers that inspect the free list)."""
        return torch.tensor(list(self._free_pages), dtype=torch.int32, device=self.device)

    def match_req(self, req):
        input_len = req.input_len
        assert input_len > 0, "Input length must be greater than 0."
        # the last prompt token is never served from the cache: its logits are needed
        return self.manager.match_prefix(req.input_ids[: input_len - 1])

    @property
    def available_size(self) -> int:
        """Tokens that can still be stored: evictable cached tokens plus the free pages."""
        return self.manager.size_info.evictable_size + len(self._free_pages) * self.page_size

    def lock(self, handle: BaseCacheHandle) -> None:
        self.manager.lock_handle(handle, unlock=False)

    def unlock(self, handle: BaseCacheHandle) -> None:
        self.manager.lock_handle(handle, unlock=True)

    def _take_pages(self, n: int) -> List[int]:
        if n > len(self._free_pages):
            evicted = self.manager.evict((n - len(self._free_pages)) * self.page_size)
            self._free(evicted)
            assert len(self._free_pages) >= n, "Eviction did not free enough space."
        return [self._free_pages.popleft() for _ in range(n)]

    def allocate(self, needed_len: int, *, start: int = 0, last_slot: Optional[int] = None) -> torch.Tensor:
        """Slots for ``needed_len`` new tokens.  With pages, the tokens are positions
        ``[start, start + needed_len)`` of their request: those that still fit the request's last
        page continue it (``last_slot`` = slot of position ``start - 1``), the rest open new
        pages.  ``page_size`` 1 ignores both keywords (the reference's signature)."""
        ps = self.page_size
        if ps == 1:
            return torch.tensor(self._take_pages(needed_len), dtype=torch.int32, device=self.device)
        head = 0 if start % ps == 0 else min(needed_len, ps - start % ps)
        parts = []
        if head:
            assert last_slot is not None and (int(last_slot) + 1) % ps == start % ps, \
                "a request that continues a page must say where its last token sits"
            parts.append(torch.arange(int(last_slot) + 1, int(last_slot) + 1 + head, dtype=torch.int32))
        rest = needed_len - head
        if rest > 0:
            pages = torch.tensor(self._take_pages(-(-rest // ps)), dtype=torch.int32)
            parts.append((pages[:, None] * ps + torch.arange(ps, dtype=torch.int32)[None]).reshape(-1)[:rest])
        out = torch.cat(parts) if parts else torch.zeros(0, dtype=torch.int32)
        return out.to(self.device)

    def free_and_cache_finished_req(self, old_handle: BaseCacheHandle, input_ids,
                                    indices: torch.Tensor) -> None:
        in_cache_len = self.manager.insert_prefix(input_ids, indices)
        # slots of tokens another request cached in the meantime are duplicates: give them back
        self._free(indices[old_handle.cached_len:in_cache_len])
        whole = len(indices) // self.page_size * self.page_size
        if in_cache_len <= whole < len(indices):
            self._free(indices[whole:])        # the partial last page is not cached
        self.unlock(old_handle)

    def check_integrity(self) -> None:
        self.manager.check_integrity()
        if len(self._free_pages) * self.page_size + self.manager.size_info.total_size != \
                self.num_pages * self.page_size:
            raise RuntimeError(
                "CacheManager integrity check failed:"
                f" free_pages({len(self._free_pages)}) * page_size({self.page_size}) +"
                f" total_size({self.manager.size_info.total_size}) != "
                f"num_pages({self.num_pages}) * page_size")
