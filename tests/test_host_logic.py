"""Host-side rules of the path that need no GPU: the decode split rule, the reassembly plan of
the request sharding, page-aligned allocation sizes."""
import numpy as np
import torch

from mini_sglang_mlx_b200 import parallel as P
from mini_sglang_mlx_b200.attention.backend import compute_num_kv_splits, split_chunk_tokens
from oracle import paged_attention_oracle as O


def test_reference_split_rule_is_the_oracles():
    lens = [1, 127, 128, 129, 4096, 5000, 100000]
    assert compute_num_kv_splits(lens, 8, policy="reference") == list(O.compute_num_kv_splits(lens))


def test_split_chunk_is_clamped_and_a_multiple_of_64():
    for total, hkv, batch in [(100, 8, 1), (9035, 8, 8), (9_400_000, 8, 256), (50_000, 2, 3), (4096, 4, 1)]:
        chunk = split_chunk_tokens(total, hkv, batch=batch)
        assert 256 <= chunk <= 4096 and chunk % 64 == 0


def test_a_small_batch_gets_one_wave_of_ctas():
    """296 CTA slots (two per SM): a batch that the plain rule would spread over a little more
    than one wave gets the chunk that makes it exactly one."""
    rng = np.random.default_rng(1)
    kv_lens = rng.integers(256, 2049, size=8).tolist()      # the small decode configuration
    hkv, slots = 8, 2 * 148
    chunk = split_chunk_tokens(sum(kv_lens), hkv, batch=len(kv_lens))
    splits = compute_num_kv_splits(kv_lens, hkv)
    assert splits == [min(32, max(1, -(-l // chunk))) for l in kv_lens]
    assert sum(splits) * hkv <= slots
    # a long-context batch keeps the bandwidth-oriented chunk
    assert split_chunk_tokens(9_400_000, 8, batch=256) == 4096


def test_gather_plan_puts_every_row_back_in_request_order():
    rng = np.random.default_rng(7)
    for world in (2, 3, 8):
        rows = rng.integers(1, 6, size=17).tolist()
        shards = P.assign_requests(rows, world)
        plan = P.GatherPlan(shards, rows)
        # what each rank would hold: its requests' rows, in shard order, padded to the widest shard
        starts = np.concatenate([[0], np.cumsum(rows)])
        full = torch.arange(int(starts[-1]), dtype=torch.float32).unsqueeze(1)
        gathered = torch.full((world * plan.width, 1), -1.0)
        for r, shard in enumerate(shards):
            local = torch.cat([full[starts[i]:starts[i + 1]] for i in shard]) if shard else full[:0]
            assert local.shape[0] == plan.local_rows[r] <= plan.width
            gathered[r * plan.width: r * plan.width + local.shape[0]] = local
        assert torch.equal(gathered.index_select(0, plan.index), full)


def test_head_slices_cover_the_heads_once():
    slices = P.head_slices(32, 8, 4)
    q = sorted(i for qs, _ in slices for i in range(32)[qs])
    kv = sorted(i for _, ks in slices for i in range(8)[ks])
    assert q == list(range(32)) and kv == list(range(8))
    for qs, ks in slices:       # a rank's query heads map to its own KV heads
        assert {i // 4 for i in range(32)[qs]} == set(range(8)[ks])
