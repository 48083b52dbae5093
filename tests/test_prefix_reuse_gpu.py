"""Prefix reuse end to end on the GPU: slot allocator + radix cache + page table
+ K/V scatter + paged prefill.  A request that shares a prompt prefix with a
finished one computes only its new tokens (prefix_len = matched length) over the
cached slots, and must get what a full prefill of its whole prompt gives
(the flow of mini_sglang_mlx/scheduler/prefill.py:51-107 and
scheduler/scheduler.py:297-330, without a model: K/V/Q rows are per-token
embeddings, so they depend on the token id only, as cached K/V must)."""
import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu

HQ, HKV, D, VOCAB = 8, 2, 128, 512


class _Cfg:
    head_dim, num_kv_heads, num_qo_heads = D, HKV, HQ


class _Prompt:
    def __init__(self, tokens):
        self.input_ids = np.asarray(tokens, dtype=np.int32)
        self.input_len = len(tokens)


@pytest.mark.parametrize("page_size", [1, 16])
def test_a_cached_prefix_is_reused_and_gives_the_full_prefill_result(page_size):
    """page_size 16: page-granular allocation, page-aligned prefix tree, attention through the
    page-granular operators; a match ends on a page boundary, the rest is recomputed."""
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    from mini_sglang_mlx_b200.scheduler import CacheManager, TableManager

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(7)
    emb_q = torch.randn(VOCAB, HQ, D, generator=g).bfloat16()
    emb_k = torch.randn(VOCAB, HKV, D, generator=g).bfloat16()
    emb_v = torch.randn(VOCAB, HKV, D, generator=g).bfloat16()

    ps = page_size
    num_pages, max_reqs, max_len = 1024 // ps * (4 if ps > 1 else 1), 4, 512
    pool = MHAKVCache(HKV, 1, D, num_pages * ps + 1, torch.bfloat16)
    page_table = torch.zeros((max_reqs + 1, max_len), dtype=torch.int32, device=dev)
    tm = TableManager(max_reqs, page_table)
    cm = CacheManager(dev, num_pages, page_size=ps)
    be = AttnBackend(_Cfg, pool, page_table, page_size=ps)

    rng = np.random.default_rng(3)
    shared = rng.integers(0, VOCAB, size=300).tolist()
    prompts = [shared[:200] + rng.integers(0, VOCAB, size=17).tolist(),     # nothing cached yet
               shared[:150] + rng.integers(0, VOCAB, size=60).tolist(),     # splits the first edge at 150
               shared[:200] + rng.integers(0, VOCAB, size=1).tolist(),      # one new token
               shared[:150] + rng.integers(0, VOCAB, size=333).tolist()]    # long suffix
    expect_cached = [w // ps * ps for w in [0, 150, 200, 150]]

    for tokens, want in zip(prompts, expect_cached):
        handle, cached = cm.match_req(_Prompt(tokens))
        assert handle.cached_len == want and cached.is_cuda
        cm.lock(handle)
        row = tm.allocate()
        n = len(tokens)
        page_table[row, :want] = cached
        fresh = cm.allocate(n - want, start=want)
        page_table[row, want:n] = fresh
        req = Req(table_idx=row, cached_len=want, device_len=n)
        batch = Batch(reqs=[req], phase=BatchPhase.PREFILL, out_loc=fresh)
        be.prepare_metadata(batch)
        new = torch.tensor(tokens[want:])
        out = be.forward(emb_q[new].to(dev), emb_k[new].to(dev), emb_v[new].to(dev), 0, batch)

        # what a prefill of the whole prompt gives, on a private contiguous pool
        t = torch.tensor(tokens)
        ref = O.paged_prefill_attention_oracle(
            emb_q[t], emb_k[t], emb_v[t], torch.tensor([0, n], dtype=torch.int32),
            torch.tensor([0, n], dtype=torch.int32), torch.arange(n, dtype=torch.int32),
            torch.tensor([0], dtype=torch.int32), be.sm_scale)
        assert_close_to_oracle(out, ref[want:], f"prefix reuse, cached {want} of {n}")

        cm.free_and_cache_finished_req(handle, np.asarray(tokens, np.int32), page_table[row, :n])
        tm.free(row)
        cm.check_integrity()

    # the pool holds every distinct prefix (of whole pages) once
    distinct = {tuple(p[: i + 1]) for p in prompts for i in range(len(p)) if (i + 1) % ps == 0}
    assert cm.manager.size_info.total_size == len(distinct) * ps


@pytest.mark.parametrize("page_size", [1, 16])
def test_a_random_stream_of_requests_under_eviction_pressure(page_size):
    """Thirty requests that share prefixes of three base prompts, one after the other, through a
    pool that holds about four prompts: matches are reused, the tree is evicted to make room,
    every result equals the full prefill of the whole prompt, and the allocator's books balance
    after every request."""
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    from mini_sglang_mlx_b200.scheduler import CacheManager, TableManager

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(17)
    vocab = 64
    emb_q = torch.randn(vocab, HQ, D, generator=g).bfloat16()
    emb_k = torch.randn(vocab, HKV, D, generator=g).bfloat16()
    emb_v = torch.randn(vocab, HKV, D, generator=g).bfloat16()
    ps = page_size
    num_pages = 2400 // ps
    pool = MHAKVCache(HKV, 1, D, num_pages * ps + 1, torch.bfloat16)
    page_table = torch.zeros((5, 1024), dtype=torch.int32, device=dev)
    tm = TableManager(4, page_table)
    cm = CacheManager(dev, num_pages, page_size=ps)
    be = AttnBackend(_Cfg, pool, page_table, page_size=ps)
    rng = np.random.default_rng(5 + ps)
    bases = [rng.integers(0, vocab, size=700).tolist() for _ in range(3)]
    reused = 0
    for it in range(30):
        base = bases[rng.integers(3)]
        tokens = base[: int(rng.integers(1, 600))] + rng.integers(0, vocab, size=int(rng.integers(1, 200))).tolist()
        n = len(tokens)
        handle, cached = cm.match_req(_Prompt(tokens))
        want = handle.cached_len
        assert want % ps == 0 and want < n
        reused += want > 0
        cm.lock(handle)
        row = tm.allocate()
        page_table[row, :want] = cached
        fresh = cm.allocate(n - want, start=want)
        page_table[row, want:n] = fresh
        batch = Batch(reqs=[Req(table_idx=row, cached_len=want, device_len=n)], phase=BatchPhase.PREFILL,
                      out_loc=fresh)
        be.prepare_metadata(batch)
        new = torch.tensor(tokens[want:])
        out = be.forward(emb_q[new].to(dev), emb_k[new].to(dev), emb_v[new].to(dev), 0, batch)
        t = torch.tensor(tokens)
        ref = O.paged_prefill_attention_oracle(
            emb_q[t], emb_k[t], emb_v[t], torch.tensor([0, n], dtype=torch.int32),
            torch.tensor([0, n], dtype=torch.int32), torch.arange(n, dtype=torch.int32),
            torch.tensor([0], dtype=torch.int32), be.sm_scale)
        assert_close_to_oracle(out, ref[want:], f"request {it}: cached {want} of {n}")
        cm.free_and_cache_finished_req(handle, np.asarray(tokens, np.int32), page_table[row, :n])
        tm.free(row)
        cm.check_integrity()
    assert reused >= 20
    assert cm.manager.size_info.total_size <= num_pages * ps
