"""Multi-GPU partition of the paged attention ops: one process per GPU.

Attention of different sequences is independent, and for one sequence the KV
head groups are independent (``kv_head = q_head // G``), so the work shards
with no exchange inside the kernels.  Each rank keeps its own page pool, page
table and metadata; the only collective is the reassembly of the output rows
(``all_gather`` over NCCL on GPUs, gloo on CPU ranks).  The reference is
single-device and has no counterpart of this module.

* by request (primary): ``assign_requests`` gives every rank a set of
  sequences with balanced KV work; ``gather_request_outputs`` returns all rows
  in the original request order on every rank.
* by KV-head group (fallback when there are fewer requests than ranks):
  ``head_slices`` gives rank r the q heads ``[r*Hq/n, (r+1)*Hq/n)`` and the KV
  heads they map to; ``gather_head_outputs`` concatenates along the head axis.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def assign_requests(work: Sequence[int], world_size: int) -> List[List[int]]:
    """Longest-processing-time-first assignment of request ids to ranks.

    ``work[i]`` is the cost of request i (its KV length for decode, visible
    keys x query rows for prefill).  Deterministic: ties go to the lower rank,
    and every rank's list is sorted, so all ranks compute the same plan."""
    order = sorted(range(len(work)), key=lambda i: (-work[i], i))
    loads = [0] * world_size
    shards: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        shards[r].append(i)
        loads[r] += work[i]
    return [sorted(s) for s in shards]


def head_slices(num_q_heads: int, num_kv_heads: int, world_size: int) -> List[Tuple[slice, slice]]:
    """(q-head slice, kv-head slice) per rank; needs world_size | num_kv_heads."""
    if num_kv_heads % world_size != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not split over {world_size} ranks")
    g = num_q_heads // num_kv_heads
    per = num_kv_heads // world_size
    return [(slice(r * per * g, (r + 1) * per * g), slice(r * per, (r + 1) * per))
            for r in range(world_size)]


class GatherPlan:
    """Where every request's rows sit in the all-gathered buffer: computed once per batch
    (host), then each reassembly is one collective and one row gather on the device."""

    def __init__(self, shards: List[List[int]], rows_per_request: Sequence[int], device=None):
        counts = [sum(rows_per_request[i] for i in s) for s in shards]
        self.width = max(counts) if counts else 0
        self.local_rows = counts
        starts = [0]
        for n in rows_per_request:
            starts.append(starts[-1] + n)
        src = [0] * starts[-1]
        for r, shard in enumerate(shards):
            off = r * self.width
            for i in shard:
                n = rows_per_request[i]
                for k in range(n):
                    src[starts[i] + k] = off + k
                off += n
        self.index = torch.tensor(src, dtype=torch.int64, device=device)


def gather_request_outputs(local_out: torch.Tensor, shards, rows_per_request: Sequence[int] = None,
                           group=None) -> torch.Tensor:
    """All ranks' output rows in original request order.

    ``local_out`` holds this rank's rows, requests in the order of
    ``shards[rank]``; request i owns ``rows_per_request[i]`` rows (1 for decode,
    its query length for prefill).  Shards are padded to the largest one so a
    single ``all_gather_into_tensor`` suffices.  ``shards`` may be a ``GatherPlan``
    built once for the batch (then ``rows_per_request`` is not needed)."""
    plan = shards if isinstance(shards, GatherPlan) else GatherPlan(shards, rows_per_request,
                                                                    local_out.device)
    world = dist.get_world_size(group)
    tail = local_out.shape[1:]
    if local_out.shape[0] == plan.width:
        padded = local_out.contiguous()
    else:
        padded = local_out.new_zeros((plan.width, *tail))
        padded[: local_out.shape[0]] = local_out
    gathered = local_out.new_empty((world * plan.width, *tail))
    dist.all_gather_into_tensor(gathered, padded, group=group)
    return gathered.index_select(0, plan.index.to(gathered.device))


def gather_head_outputs(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """(rows, Hq/n, D) per rank -> (rows, Hq, D) on every rank."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)
