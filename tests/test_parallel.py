"""Request / head sharding and output reassembly with two CPU ranks (gloo);
each rank computes its shard with the oracle, the gathered result must equal
the unsharded one."""
import math
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mini_sglang_mlx_b200 import parallel as P
from oracle import paged_attention_oracle as O


def test_assign_requests_balances_and_covers():
    work = [131072, 4096, 5000, 90000, 4097, 60000, 8000, 100]
    shards = P.assign_requests(work, 4)
    assert sorted(i for s in shards for i in s) == list(range(len(work)))
    loads = [sum(work[i] for i in s) for s in shards]
    assert max(loads) == 131072  # the longest request alone bounds the makespan
    assert P.assign_requests(work, 4) == shards
    assert P.assign_requests([5, 5], 4) == [[0], [1], [], []]


def test_head_slices():
    assert P.head_slices(32, 8, 4) == [(slice(0, 8), slice(0, 2)), (slice(8, 16), slice(2, 4)),
                                       (slice(16, 24), slice(4, 6)), (slice(24, 32), slice(6, 8))]
    with pytest.raises(ValueError):
        P.head_slices(32, 4, 8)


def _problem():
    g = torch.Generator().manual_seed(0)
    hq, hkv, d = 8, 2, 128
    kv_lens = [40, 7, 130, 65, 9]
    S = sum(kv_lens)
    kc = torch.randn(S, hkv, d, generator=g).bfloat16()
    vc = torch.randn(S, hkv, d, generator=g).bfloat16()
    q = torch.randn(len(kv_lens), hq, d, generator=g).bfloat16()
    slots = torch.randperm(S, generator=g).int()
    return q, kc, vc, kv_lens, slots


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, kc, vc, kv_lens, slots = _problem()
        scale = 1 / math.sqrt(128)
        indptr = torch.from_numpy(O.build_indptr(kv_lens))
        # --- by request: the rank rebuilds CSR metadata for its own sequences only
        shards = P.assign_requests(kv_lens, world)
        mine = shards[rank]
        my_lens = [kv_lens[i] for i in mine]
        my_slots = torch.cat([slots[indptr[i]:indptr[i + 1]] for i in mine]) if mine else slots[:0]
        local = O.paged_decode_attention_oracle(q[mine], kc, vc, torch.from_numpy(O.build_indptr(my_lens)),
                                                my_slots, scale)
        full = P.gather_request_outputs(local, shards, [1] * len(kv_lens))
        # --- by KV-head group
        qs, ks = P.head_slices(q.shape[1], kc.shape[1], world)[rank]
        local_h = O.paged_decode_attention_oracle(q[:, qs], kc[:, ks], vc[:, ks], indptr, slots, scale)
        full_h = P.gather_head_outputs(local_h)
        if rank == 0:
            ret["by_request"] = full
            ret["by_head"] = full_h
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reassembles_the_unsharded_result():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    q, kc, vc, kv_lens, slots = _problem()
    ref = O.paged_decode_attention_oracle(q, kc, vc, torch.from_numpy(O.build_indptr(kv_lens)), slots,
                                          1 / math.sqrt(128))
    torch.testing.assert_close(ret["by_request"], ref, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(ret["by_head"], ref, atol=1e-6, rtol=1e-6)
