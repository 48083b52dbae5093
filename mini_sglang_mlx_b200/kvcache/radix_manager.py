"""Radix-tree prefix cache over per-token slot ids.

Same contract as the reference's ``RadixCacheManager``
(mini_sglang_mlx/kvcache/radix_manager.py:98-275): ``match_prefix`` returns
the slot ids of the longest cached prefix (splitting an edge at the match
point), ``insert_prefix`` adds the uncached tail, ``lock_handle`` moves a
path between the evictable and the protected size, ``evict`` drops
least-recently-used unlocked leaves.  Token keys live in host memory (numpy)
so that walking the tree never touches the device; slot ids are int32
tensors on the pool's device, so a match can be written into the page table
without a host round trip.  The edge comparison is ``fast_compare_key``.
Recency is a logical clock (one tick per walk), which keeps eviction order
deterministic.  The hybrid (recurrent-state) variant of the reference is not
built: it belongs to a model family outside the attention path.

``page_size`` > 1 (the reference hard-wires 1, mini_sglang_mlx/engine/engine.py:103) keeps the
tree page-aligned so that the page-granular attention entries can use what it returns: every
edge holds whole pages, an edge is split only at a page boundary (a match that ends inside a
page is rounded down: that page is recomputed, not shared), only the whole pages of a finished
request are inserted, and children are told apart by their first PAGE of tokens (two edges
may agree on their first token and differ later in the page).
"""
from __future__ import annotations

import heapq
import itertools
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..kernel import fast_compare_key
from .base import BaseCacheHandle, SizeInfo


class RadixTreeNode:
    __slots__ = ("children", "parent", "ref_count", "timestamp", "key", "value", "uid")
    _uids = itertools.count()

    def __init__(self, timestamp: int) -> None:
        self.children: Dict[int, "RadixTreeNode"] = {}
        self.parent: Optional["RadixTreeNode"] = None
        self.ref_count = 0
        self.timestamp = timestamp
        self.key: np.ndarray = np.zeros(0, dtype=np.int32)       # token ids on this edge
        self.value: torch.Tensor = torch.zeros(0, dtype=torch.int32)  # their slot ids
        self.uid = next(RadixTreeNode._uids)

    @property
    def length(self) -> int:
        return int(self.key.shape[0])

    def is_root(self) -> bool:
        return self.parent is None

    def is_leaf(self) -> bool:
        return not self.children

    def attach(self, parent: "RadixTreeNode", page_size: int = 1) -> None:
        self.parent = parent
        parent.children[_child_key(self.key, 0, page_size)] = self

    def __lt__(self, other: "RadixTreeNode") -> bool:  # heap order: least recently used first
        return (self.timestamp, self.uid) < (other.timestamp, other.uid)


@dataclass(frozen=True)
class RadixCacheHandle(BaseCacheHandle):
    node: RadixTreeNode


def _child_key(key: np.ndarray, pos: int, page_size: int):
    """What a node's children are indexed by: the first token of the edge, or its first page."""
    if page_size == 1:
        return int(key[pos])
    return key[pos:pos + page_size].tobytes()


def _as_key(input_ids) -> np.ndarray:
    if isinstance(input_ids, torch.Tensor):
        input_ids = input_ids.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(input_ids).reshape(-1), dtype=np.int32)


class RadixCacheManager:
    def __init__(self, device=None, page_size: int = 1) -> None:
        assert page_size >= 1
        self.page_size = page_size
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.empty_tensor = torch.zeros(0, dtype=torch.int32, device=self.device)
        self._clock = itertools.count(1)
        self.root_node = RadixTreeNode(0)
        self.root_node.ref_count = 1  # the root is never evicted
        self.evictable_size = 0
        self.protected_size = 0

    # ------------------------------------------------------------------ queries
    def _whole_pages(self, key: np.ndarray) -> np.ndarray:
        return key if self.page_size == 1 else key[: key.shape[0] // self.page_size * self.page_size]

    def match_prefix(self, input_ids) -> Tuple[RadixCacheHandle, torch.Tensor]:
        node, matched = self._walk(self._whole_pages(_as_key(input_ids)))
        if matched == 0:
            return RadixCacheHandle(0, self.root_node), self.empty_tensor
        parts: List[torch.Tensor] = []
        cur = node
        while not cur.is_root():
            parts.append(cur.value)
            cur = cur.parent
        parts.reverse()
        return RadixCacheHandle(matched, node), torch.cat(parts)

    @property
    def size_info(self) -> SizeInfo:
        return SizeInfo(self.evictable_size, self.protected_size)

    # ------------------------------------------------------------------ updates
    def lock_handle(self, handle: BaseCacheHandle, unlock: bool = False) -> None:
        assert isinstance(handle, RadixCacheHandle)
        node = handle.node
        while not node.is_root():
            if unlock:
                node.ref_count -= 1
                assert node.ref_count >= 0
                if node.ref_count == 0:
                    self.evictable_size += node.length
                    self.protected_size -= node.length
            else:
                if node.ref_count == 0:
                    self.evictable_size -= node.length
                    self.protected_size += node.length
                node.ref_count += 1
            node = node.parent

    def insert_prefix(self, input_ids, indices: torch.Tensor) -> int:
        key = _as_key(input_ids)
        assert indices.shape[0] == key.shape[0], "one slot id per token"
        key = self._whole_pages(key)          # a trailing partial page is not cached
        node, matched = self._walk(key)
        if matched < key.shape[0]:
            leaf = RadixTreeNode(next(self._clock))
            leaf.key = key[matched:].copy()
            leaf.value = indices[matched:key.shape[0]].to(device=self.device,
                                                          dtype=torch.int32).reshape(-1).clone()
            leaf.attach(node, self.page_size)
            self.evictable_size += leaf.length
        return matched

    def evict(self, size: int) -> torch.Tensor:
        if size == 0:
            return self.empty_tensor
        assert size <= self.evictable_size, \
            f"Cannot evict {size}, only {self.evictable_size} is evictable"
        heap = [n for n in self._nodes() if n.is_leaf() and n.ref_count == 0 and not n.is_root()]
        heapq.heapify(heap)
        freed: List[torch.Tensor] = []
        got = 0
        while got < size:
            assert heap, f"Cannot evict enough cache, need {size}, only {got} evicted"
            node = heapq.heappop(heap)
            got += node.length
            freed.append(node.value)
            self.evictable_size -= node.length
            parent = node.parent
            del parent.children[_child_key(node.key, 0, self.page_size)]
            if parent.is_leaf() and parent.ref_count == 0 and not parent.is_root():
                heapq.heappush(heap, parent)
        return torch.cat(freed)

    def reset(self) -> None:
        raise NotImplementedError("RadixCacheManager.reset is not implemented")

    def check_integrity(self) -> None:
        evictable = protected = 0
        for node in self._nodes():
            if node.is_root():
                continue
            assert node.length > 0 and node.value.shape[0] == node.length
            assert node.length % self.page_size == 0, "an edge that does not hold whole pages"
            assert node.parent.children.get(_child_key(node.key, 0, self.page_size)) is node
            assert all(c.ref_count <= node.ref_count for c in node.children.values()), \
                "a locked node below an unlocked one"
            if node.ref_count == 0:
                evictable += node.length
            else:
                protected += node.length
        if (evictable, protected) != (self.evictable_size, self.protected_size):
            raise RuntimeError(
                f"radix cache accounting is off: counted ({evictable}, {protected}), "
                f"recorded ({self.evictable_size}, {self.protected_size})")

    # ------------------------------------------------------------------ internals
    def _nodes(self):
        stack = [self.root_node]
        while stack:
            node = stack.pop()
            yield node
            stack.extend(node.children.values())

    def _split(self, node: RadixTreeNode, pos: int) -> RadixTreeNode:
        """Cut the edge into node at `pos`: a new upper node takes key[:pos]; returns it."""
        assert 0 < pos < node.length
        upper = RadixTreeNode(node.timestamp)
        upper.key, upper.value = node.key[:pos].copy(), node.value[:pos]
        upper.ref_count = node.ref_count
        upper.attach(node.parent, self.page_size)
        node.key, node.value = node.key[pos:].copy(), node.value[pos:]
        node.attach(upper, self.page_size)
        return upper

    def _walk(self, key: np.ndarray) -> Tuple[RadixTreeNode, int]:
        """Deepest node whose path is a prefix of `key` (edges are split at a partial match)
        and the number of tokens matched; refreshes the recency of fully matched nodes."""
        tick = next(self._clock)
        node, matched, n = self.root_node, 0, key.shape[0]
        ps = self.page_size
        while matched + ps <= n:
            child = node.children.get(_child_key(key, matched, ps))
            if child is None:
                break
            m = fast_compare_key(child.key, key[matched:]) // ps * ps   # whole pages only
            matched += m
            if m < child.length:
                return self._split(child, m), matched    # m >= ps: the first page is the child key
            child.timestamp = tick
            node = child
        return node, matched
