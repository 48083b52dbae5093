"""Brute-force model of the prefix cache (TEST INFRASTRUCTURE ONLY).

What the reference's radix tree promises
(mini_sglang_mlx/kvcache/radix_manager.py:130-156; pinned by
mini_sglang_mlx/tests/test_radix_prefix_cache.py:46-54 and
tests/_factories.py:111-118): ``match_prefix`` returns the slot ids that were
stored for the longest cached prefix of the query, and the first request to
cache a token position owns its slot (a later insert of the same prefix keeps
the old slots and reports how many tokens were already there).  This model
keeps one dictionary entry per cached prefix instead of a tree, so it has no
edges to split and no structure to get wrong.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


class PrefixCacheModel:
    """``page_size`` > 1 is the page-aligned variant of this build (the reference has one token
    per page): a prefix is cached, matched and shared in whole pages only, so the model keeps one
    entry per cached prefix of whole pages."""

    def __init__(self, page_size: int = 1) -> None:
        self.page_size = page_size
        self.slots_of: Dict[Tuple[int, ...], List[int]] = {}   # prefix -> slots of its last page

    def match(self, tokens: Sequence[int]) -> List[int]:
        out: List[int] = []
        ps = self.page_size
        for end in range(ps, len(tokens) + 1, ps):
            slots = self.slots_of.get(tuple(tokens[:end]))
            if slots is None:
                break
            out.extend(slots)
        return out

    def insert(self, tokens: Sequence[int], slots: Sequence[int]) -> int:
        """Returns how many leading tokens were cached already (their slots are kept)."""
        ps = self.page_size
        already = len(self.match(tokens))
        for end in range(already + ps, len(tokens) + 1, ps):
            self.slots_of[tuple(tokens[:end])] = [int(x) for x in slots[end - ps:end]]
        return already

    @property
    def size(self) -> int:
        return len(self.slots_of) * self.page_size
