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
    def __init__(self) -> None:
        self.slot_of: Dict[Tuple[int, ...], int] = {}   # prefix -> slot of its last token

    def match(self, tokens: Sequence[int]) -> List[int]:
        out: List[int] = []
        for i in range(len(tokens)):
            slot = self.slot_of.get(tuple(tokens[: i + 1]))
            if slot is None:
                break
            out.append(slot)
        return out

    def insert(self, tokens: Sequence[int], slots: Sequence[int]) -> int:
        """Returns how many leading tokens were cached already (their slots are kept)."""
        already = len(self.match(tokens))
        for i in range(already, len(tokens)):
            self.slot_of[tuple(tokens[: i + 1])] = int(slots[i])
        return already

    @property
    def size(self) -> int:
        return len(self.slot_of)
