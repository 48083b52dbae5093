"""Prefix cache, slot allocator and table manager (host logic, CPU tensors).

The invariants are the ones the reference's weight-free tests pin
(mini_sglang_mlx/tests/test_radix_prefix_cache.py, tests/_factories.py:111-118,
tests/test_scheduler_loop.py:195-214): a match returns exactly the cached slot
ids, a match is a pure query, locking moves a prefix out of the evictable
size, eviction is least-recently-used and never touches a locked path, and
free + cached slots always add up to the pool.
"""
import numpy as np
import pytest
import torch

from mini_sglang_mlx_b200 import fast_compare_key
from mini_sglang_mlx_b200.kvcache import RadixCacheManager, create_cache_manager
from mini_sglang_mlx_b200.scheduler import CacheManager, TableManager
from oracle.prefix_cache_oracle import PrefixCacheModel


def ids(*tokens):
    return np.asarray(tokens, dtype=np.int32)


def cache_prefix(cm: CacheManager, tokens):
    """What a finished request does: allocate slots, hand them to the prefix cache."""
    handle, cached = cm.manager.match_prefix(ids(*tokens))
    cm.lock(handle)
    fresh = cm.allocate(len(tokens) - handle.cached_len)
    slots = torch.cat([cached, fresh])
    cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
    cm.check_integrity()
    return slots


# ------------------------------------------------------------------ fast_compare_key
@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_fast_compare_key(dtype):
    a = np.arange(1000, dtype=dtype)
    for cut in (0, 1, 7, 8, 9, 500, 999):
        b = a.copy()
        b[cut] = -1
        assert fast_compare_key(a, b) == cut
        assert fast_compare_key(a[: cut + 1], b) == cut
    assert fast_compare_key(a, a[:123]) == 123
    assert fast_compare_key(a[:0], a) == 0
    assert fast_compare_key(torch.from_numpy(a), torch.from_numpy(a.copy())) == 1000


def test_fast_compare_key_rejects_bad_inputs():
    a = np.arange(4, dtype=np.int32)
    with pytest.raises(RuntimeError, match="same dtype"):
        fast_compare_key(a, a.astype(np.int64))
    with pytest.raises(RuntimeError, match="int32 or int64"):
        fast_compare_key(a.astype(np.int16), a.astype(np.int16))
    with pytest.raises(RuntimeError, match="1D"):
        fast_compare_key(a.reshape(2, 2), a.reshape(2, 2))
    with pytest.raises(RuntimeError, match="contiguous"):
        fast_compare_key(np.arange(8, dtype=np.int32)[::2], a)


# ------------------------------------------------------------------ radix tree
def test_match_returns_exactly_the_cached_slots_and_is_a_pure_query():
    cm = CacheManager("cpu", 64)
    slots = cache_prefix(cm, [1, 2, 3, 4, 5, 6])
    before = (cm.manager.size_info, cm.available_size)
    for _ in range(3):
        handle, got = cm.manager.match_prefix(ids(1, 2, 3, 4, 5, 6, 7))
        assert handle.cached_len == 6
        assert got.tolist() == slots.tolist()
        assert (cm.manager.size_info, cm.available_size) == before


def test_partial_match_splits_the_edge_and_keeps_the_slots():
    cm = CacheManager("cpu", 64)
    slots = cache_prefix(cm, [1, 2, 3, 4, 5, 6])
    handle, got = cm.manager.match_prefix(ids(1, 2, 3, 9))
    assert handle.cached_len == 3 and got.tolist() == slots[:3].tolist()
    assert handle.node.length == 3 and not handle.node.is_leaf()
    other = cache_prefix(cm, [1, 2, 3, 9, 10])
    assert other[:3].tolist() == slots[:3].tolist()          # shared prefix, same slots
    _, full = cm.manager.match_prefix(ids(1, 2, 3, 4, 5, 6))
    assert full.tolist() == slots.tolist()
    assert cm.manager.size_info.total_size == 6 + 2


def test_insert_reports_what_was_cached_already_and_duplicates_are_freed():
    cm = CacheManager("cpu", 32)
    cache_prefix(cm, [5, 6, 7, 8])
    free_before = len(cm._free_slots)
    # a second request computed the same prompt without a cache hit (it started earlier)
    handle, _ = cm.manager.match_prefix(ids())            # matched nothing at admission
    cm.lock(handle)
    dup = cm.allocate(4)
    cm.free_and_cache_finished_req(handle, ids(5, 6, 7, 8), dup)
    assert len(cm._free_slots) == free_before             # its four slots came back
    cm.check_integrity()


def test_locking_moves_the_prefix_out_of_the_evictable_size():
    cm = CacheManager("cpu", 32)
    cache_prefix(cm, [1, 2, 3, 4, 5, 6])
    handle, _ = cm.manager.match_prefix(ids(1, 2, 3, 4, 5, 6))
    before = cm.available_size
    cm.lock(handle)
    assert cm.available_size == before - 6
    assert cm.manager.size_info.protected_size == 6
    with pytest.raises(AssertionError):
        cm.manager.evict(1)                               # nothing evictable
    cm.unlock(handle)
    assert cm.available_size == before
    cm.check_integrity()


def test_eviction_is_least_recently_used_and_returns_the_slots():
    cm = CacheManager("cpu", 12)
    a = cache_prefix(cm, [1, 2, 3])
    b = cache_prefix(cm, [10, 11, 12])
    c = cache_prefix(cm, [20, 21, 22])
    cm.manager.match_prefix(ids(1, 2, 3))                 # touch A: B is now the coldest
    assert len(cm._free_slots) == 3
    got = cm.allocate(5)                                  # needs 2 more than free: evicts B (3)
    assert set(b.tolist()) <= set(got.tolist()) | set(cm._free_slots.tolist())
    assert cm.manager.match_prefix(ids(10, 11, 12))[0].cached_len == 0
    assert cm.manager.match_prefix(ids(1, 2, 3))[0].cached_len == 3
    assert cm.manager.match_prefix(ids(20, 21, 22))[0].cached_len == 3
    cm._free(got)
    cm.check_integrity()
    del a, c


def test_eviction_never_takes_a_locked_path_and_cascades_to_parents():
    cm = CacheManager("cpu", 16)
    cache_prefix(cm, [1, 2, 3, 4])
    cache_prefix(cm, [1, 2, 7, 8])                        # splits at [1, 2]
    handle, _ = cm.manager.match_prefix(ids(1, 2, 3, 4))
    cm.lock(handle)
    assert cm.manager.size_info == (2, 4)                 # only the [7, 8] leaf is evictable
    evicted = cm.manager.evict(2)
    assert len(evicted) == 2
    assert cm.manager.match_prefix(ids(1, 2, 7, 8))[0].cached_len == 2
    cm._free(evicted)
    cm.unlock(handle)
    # now everything can go: the leaf first, then its parent [1, 2] once it is a leaf
    evicted = cm.manager.evict(4)
    assert len(evicted) == 4 and cm.manager.root_node.is_leaf()
    cm._free(evicted)
    cm.check_integrity()
    assert len(cm._free_slots) == 16


def test_evicting_more_than_evictable_is_refused():
    cm = CacheManager("cpu", 8)
    cache_prefix(cm, [1, 2, 3])
    with pytest.raises(AssertionError, match="only 3 is evictable"):
        cm.manager.evict(4)
    assert cm.manager.evict(0).numel() == 0


def test_random_inserts_and_matches_agree_with_the_brute_force_model():
    rng = np.random.default_rng(0)
    cm = CacheManager("cpu", 100000)
    model = PrefixCacheModel()
    stems = [list(rng.integers(0, 5, size=rng.integers(1, 12))) for _ in range(8)]
    for step in range(300):
        stem = stems[rng.integers(len(stems))]
        tokens = stem[: rng.integers(1, len(stem) + 1)] + list(rng.integers(0, 5, size=rng.integers(0, 6)))
        if rng.random() < 0.5:
            handle, cached = cm.manager.match_prefix(ids(*tokens))
            assert cached.tolist() == model.match(tokens), f"step {step}"
            assert handle.cached_len == len(cached)
        else:
            handle, cached = cm.manager.match_prefix(ids(*tokens))
            cm.lock(handle)
            fresh = cm.allocate(len(tokens) - handle.cached_len)
            slots = torch.cat([cached, fresh])
            already = model.insert(tokens, slots.tolist())
            assert already >= handle.cached_len
            cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
        cm.check_integrity()
        assert cm.manager.size_info.total_size == model.size


def test_naive_manager_caches_nothing():
    m = create_cache_manager(type="naive")
    handle, got = m.match_prefix(ids(1, 2, 3))
    assert handle.cached_len == 0 and got.numel() == 0
    assert m.insert_prefix(ids(1, 2), torch.tensor([4, 5], dtype=torch.int32)) == 2
    assert m.size_info.total_size == 0


# ------------------------------------------------------------------ a scheduler-shaped loop
class _Pending:
    def __init__(self, tokens):
        self.input_ids = ids(*tokens)
        self.input_len = len(tokens)


def test_requests_sharing_prefixes_under_memory_pressure_keep_the_books_balanced():
    """Admission (match, lock, table row, copy matched slots, allocate the rest), completion
    (cache and unlock) and eviction, checking after every step that free + cached slots
    equal the pool and that a page-table row holds the request's slots in order."""
    rng = np.random.default_rng(1)
    num_pages, max_reqs, max_len = 256, 4, 64
    cm = CacheManager("cpu", num_pages)
    page_table = torch.zeros((max_reqs + 1, max_len), dtype=torch.int32)
    tm = TableManager(max_reqs, page_table)
    system = list(rng.integers(0, 1000, size=20))
    running = []
    for step in range(200):
        if running and (len(running) == max_reqs or rng.random() < 0.4):
            row, handle, tokens, slots = running.pop(int(rng.integers(len(running))))
            assert page_table[row, : len(tokens)].tolist() == slots.tolist()
            cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
            tm.free(row)
        else:
            tokens = system[: rng.integers(1, 21)] + list(rng.integers(0, 1000, size=rng.integers(1, 30)))
            handle, cached = cm.match_req(_Pending(tokens))
            assert handle.cached_len <= len(tokens) - 1     # the last token is always computed
            cm.lock(handle)
            need = len(tokens) - handle.cached_len
            if need > cm.available_size:
                cm.unlock(handle)
                continue
            row = tm.allocate()
            fresh = cm.allocate(need)
            slots = torch.cat([cached, fresh])
            page_table[row, : len(tokens)] = slots
            assert len(set(slots.tolist())) == len(tokens)  # a request never holds a slot twice
            running.append((row, handle, tokens, slots))
        cm.manager.check_integrity()
        if not running:
            cm.check_integrity()      # holds when idle: every slot is free or cached
        held = sum(len(r[3]) - r[1].cached_len for r in running)
        assert len(cm._free_slots) + cm.manager.size_info.total_size + held == num_pages
    assert tm.available_size == max_reqs - len(running)


# ------------------------------------------------------------------ page-aligned variant
# The reference allocates single tokens and splits radix edges anywhere
# (mini_sglang_mlx/scheduler/cache.py:45-57, kvcache/radix_manager.py:73-87); with pages of 16
# tokens the same invariants hold in whole pages.
PS = 16


def paged_cache_prefix(cm: CacheManager, tokens):
    """A finished request under page-granular allocation: matched whole pages are shared, the
    rest is computed into fresh pages, then the request hands its slots over."""
    handle, cached = cm.manager.match_prefix(ids(*tokens))
    cm.lock(handle)
    assert handle.cached_len % PS == 0
    fresh = cm.allocate(len(tokens) - handle.cached_len, start=handle.cached_len)
    slots = torch.cat([cached, fresh])
    # token t of a request sits at page(t // PS) * PS + t % PS
    assert all(int(slots[t]) % PS == t % PS for t in range(len(tokens)))
    assert all(int(slots[t]) // PS == int(slots[t // PS * PS]) // PS for t in range(len(tokens)))
    cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
    cm.check_integrity()
    return slots


def test_paged_match_is_whole_pages_and_a_partial_page_is_recomputed():
    cm = CacheManager("cpu", 64, page_size=PS)
    tokens = list(range(100, 140))                            # 2 whole pages + 8 tokens
    slots = paged_cache_prefix(cm, tokens)
    assert cm.manager.size_info.total_size == 32              # the partial page was not cached ...
    assert len(cm._free_slots) == 64 - 2                      # ... and its page came back
    handle, got = cm.manager.match_prefix(ids(*tokens, 7))
    assert handle.cached_len == 32 and got.tolist() == slots[:32].tolist()
    # a query that leaves the cached prefix inside the second page shares the first page only
    handle, got = cm.manager.match_prefix(ids(*(tokens[:20] + [1, 2, 3] * 10)))
    assert handle.cached_len == 16 and got.tolist() == slots[:16].tolist()
    assert handle.node.length == 16                           # the edge was cut at the page boundary
    # fewer tokens than a page can never match
    assert cm.manager.match_prefix(ids(*tokens[:15]))[0].cached_len == 0
    cm.check_integrity()


def test_paged_children_that_share_their_first_token_are_told_apart_by_the_page():
    cm = CacheManager("cpu", 64, page_size=PS)
    a = list(range(16)) + list(range(100, 116))
    b = list(range(16)) + [100] + list(range(200, 215))       # same first token in the second page
    sa = paged_cache_prefix(cm, a)
    sb = paged_cache_prefix(cm, b)
    assert sb[:16].tolist() == sa[:16].tolist()               # first page shared
    assert set(sb[16:].tolist()).isdisjoint(sa[16:].tolist())
    assert cm.manager.match_prefix(ids(*a))[1].tolist() == sa.tolist()
    assert cm.manager.match_prefix(ids(*b))[1].tolist() == sb.tolist()
    assert cm.manager.size_info.total_size == 48


def test_paged_allocation_continues_the_last_page_before_it_opens_a_new_one():
    cm = CacheManager("cpu", 8, page_size=PS)
    first = cm.allocate(20)                                   # positions 0..19: one page + 4 tokens
    assert first.tolist() == list(range(0, 16)) + list(range(16, 20))
    more = cm.allocate(14, start=20, last_slot=int(first[-1]))  # 12 fit the second page, 2 open a third
    assert more.tolist() == list(range(20, 32)) + [32, 33]
    one = cm.allocate(1, start=34, last_slot=int(more[-1]))   # a decode step inside a page: no new page
    assert one.tolist() == [34] and len(cm._free_slots) == 5
    with pytest.raises(AssertionError):
        cm.allocate(3, start=35)                              # continuing a page needs its last slot
    # verify slab of K+1 = 8 tokens from a page boundary: one fresh page
    slab = cm.allocate(8, start=48)
    assert slab.tolist() == list(range(48, 56))


def test_paged_eviction_returns_whole_pages():
    cm = CacheManager("cpu", 6, page_size=PS)
    a = paged_cache_prefix(cm, list(range(32)))
    b = paged_cache_prefix(cm, list(range(1000, 1032)))
    cm.manager.match_prefix(ids(*range(32)))                  # touch A: B is the coldest
    assert len(cm._free_slots) == 2
    got = cm.allocate(3 * PS + 5)                             # 4 pages: evicts B's two
    assert len(got) == 3 * PS + 5 and len(cm._free_slots) == 0
    assert cm.manager.match_prefix(ids(*range(1000, 1032)))[0].cached_len == 0
    assert cm.manager.match_prefix(ids(*range(32)))[0].cached_len == 32
    assert {int(s) // PS for s in got.tolist()} >= {int(s) // PS for s in b.tolist()}
    del a


def test_paged_random_inserts_and_matches_agree_with_the_brute_force_model():
    rng = np.random.default_rng(3)
    cm = CacheManager("cpu", 4096, page_size=PS)
    model = PrefixCacheModel(page_size=PS)
    stems = [list(rng.integers(0, 3, size=rng.integers(PS, 6 * PS))) for _ in range(6)]
    for step in range(300):
        stem = stems[rng.integers(len(stems))]
        tokens = stem[: rng.integers(1, len(stem) + 1)] + list(rng.integers(0, 3, size=rng.integers(0, 2 * PS)))
        handle, cached = cm.manager.match_prefix(ids(*tokens))
        assert cached.tolist() == model.match(tokens), f"step {step}"
        assert handle.cached_len == len(cached) and handle.cached_len % PS == 0
        if rng.random() < 0.5:
            cm.lock(handle)
            fresh = cm.allocate(len(tokens) - handle.cached_len, start=handle.cached_len)
            slots = torch.cat([cached, fresh])
            already = model.insert(tokens, slots.tolist())
            assert already >= handle.cached_len
            cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
        cm.check_integrity()
        assert cm.manager.size_info.total_size == model.size


def test_paged_scheduler_shaped_loop_keeps_the_books_balanced():
    """The loop of the token-granular test above with pages of 16 tokens, plus decode steps that
    grow a running request by one token (filling its last page before a new one is taken)."""
    rng = np.random.default_rng(5)
    num_pages, max_reqs, max_len = 64, 4, 160
    cm = CacheManager("cpu", num_pages, page_size=PS)
    page_table = torch.zeros((max_reqs + 1, max_len), dtype=torch.int32)
    tm = TableManager(max_reqs, page_table)
    system = list(rng.integers(0, 1000, size=40))
    running = []
    for step in range(300):
        r = rng.random()
        if running and (len(running) == max_reqs or r < 0.3):
            row, handle, tokens, slots = running.pop(int(rng.integers(len(running))))
            assert page_table[row, : len(tokens)].tolist() == slots.tolist()
            cm.free_and_cache_finished_req(handle, ids(*tokens), slots)
            tm.free(row)
        elif running and r < 0.6:
            i = int(rng.integers(len(running)))
            row, handle, tokens, slots = running[i]
            if len(tokens) < max_len and cm.available_size >= PS:
                new = cm.allocate(1, start=len(tokens), last_slot=int(slots[-1]))
                assert int(new[0]) % PS == len(tokens) % PS
                slots = torch.cat([slots, new])
                tokens = tokens + [int(rng.integers(0, 1000))]
                page_table[row, len(tokens) - 1] = new[0]
                running[i] = (row, handle, tokens, slots)
        else:
            tokens = system[: rng.integers(1, 41)] + list(rng.integers(0, 1000, size=rng.integers(1, 40)))
            handle, cached = cm.match_req(_Pending(tokens))
            assert handle.cached_len <= len(tokens) - 1 and handle.cached_len % PS == 0
            cm.lock(handle)
            need = len(tokens) - handle.cached_len
            if need + PS > cm.available_size:
                cm.unlock(handle)
                continue
            row = tm.allocate()
            fresh = cm.allocate(need, start=handle.cached_len)
            slots = torch.cat([cached, fresh])
            page_table[row, : len(tokens)] = slots
            assert len(set(slots.tolist())) == len(tokens)
            running.append((row, handle, tokens, slots))
        cm.manager.check_integrity()
        if not running:
            cm.check_integrity()
        held_pages = sum(-(-(len(r[3]) - r[1].cached_len) // PS) for r in running)
        assert (len(cm._free_slots) + held_pages) * PS + cm.manager.size_info.total_size == num_pages * PS
