"""Paged decode attention on the GPU (through the C-ABI) against the fp32 oracle.

Shape lists follow the reference's sweeps
(mini-sglang-mlx-kernel/test_and_bench/paged_decode_attention.py:18-23, 288,
303-309) at head_dim 128, plus what it never covers: permuted slots, page
size 16 layouts, shared prefix pages, split-count invariance, empty rows.
"""
import math

import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu

HEAD_CONFIGS = [(2, 16), (4, 16), (4, 24), (2, 32), (8, 16), (8, 32), (1, 1), (4, 4)]  # (Hkv, Hq)
SINGLE_LENS = [1, 237, 512, 809, 1024, 2048, 3333, 4096, 8192]
RAGGED = [[1, 237], [512, 1024, 2048], [237, 809, 3333, 4096], [1] * 8, [4096] * 4]


def make_inputs(kv_lens, hkv, hq, *, permute=True, seed=0, d=128, extra_slots=7, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    total = sum(kv_lens)
    S = total + extra_slots
    kc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    q = torch.randn(len(kv_lens), hq, d, generator=g).to(dtype).cuda()
    slots = (torch.randperm(S, generator=g)[:total] if permute else torch.arange(total)).int().cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
    return q, kc, vc, indptr, slots, splits


def run(q, kc, vc, indptr, slots, splits, max_splits=32):
    from mini_sglang_mlx_b200 import paged_decode_attention
    out = paged_decode_attention(q, kc, vc, indptr, slots, splits, 1 / math.sqrt(q.shape[-1]), max_splits)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("hkv,hq", HEAD_CONFIGS)
@pytest.mark.parametrize("kv_len", SINGLE_LENS)
def test_single_sequence(hkv, hq, kv_len):
    args = make_inputs([kv_len], hkv, hq, seed=kv_len)
    out = run(*args)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(out, ref, f"decode L={kv_len} Hkv={hkv} Hq={hq}")


@pytest.mark.parametrize("hkv,hq", HEAD_CONFIGS[:6])
@pytest.mark.parametrize("kv_lens", RAGGED, ids=[str(r) for r in RAGGED])
def test_ragged_batch(hkv, hq, kv_lens):
    args = make_inputs(kv_lens, hkv, hq, seed=len(kv_lens))
    out = run(*args)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(out, ref, f"decode {kv_lens}")


REF_HEAD_CONFIGS_D256 = [(2, 16), (4, 16), (4, 24), (2, 32)]  # the reference's own sweep (head_dim 256)


@pytest.mark.parametrize("hkv,hq", REF_HEAD_CONFIGS_D256)
@pytest.mark.parametrize("kv_lens", [[1], [237], [809], [4096], [8192], [1, 237], [237, 809, 3333, 4096]],
                         ids=lambda v: str(v))
def test_head_dim_256_reference_sweep(hkv, hq, kv_lens):
    """Shapes of mini-sglang-mlx-kernel/test_and_bench/paged_decode_attention.py:18-23, 288, 303-309
    (identity slots there; permuted here)."""
    args = make_inputs(kv_lens, hkv, hq, seed=sum(kv_lens), d=256)
    out = run(*args)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(256))
    assert_close_to_oracle(out, ref, f"decode D=256 {kv_lens} Hkv={hkv} Hq={hq}")


def test_identity_mapping_as_the_reference_tests_use():
    args = make_inputs([809, 3333], 4, 16, permute=False)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(run(*args), ref, "identity slots")


@pytest.mark.parametrize("kv_len", [63, 64, 65, 127, 128, 129, 255, 257, 4095, 4097])
def test_split_and_tile_boundaries(kv_len):
    args = make_inputs([kv_len, 1, kv_len + 1], 2, 8, seed=kv_len)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(run(*args), ref, f"boundary L={kv_len}")


def test_short_lengths_exhaustive():
    lens = list(range(1, 81))
    args = make_inputs(lens, 2, 4, seed=11)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(run(*args), ref, "L=1..80")


def test_result_does_not_depend_on_the_split_hint():
    q, kc, vc, indptr, slots, _ = make_inputs([5000, 300, 2049], 4, 16, seed=3)
    ref = O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, 1 / math.sqrt(128))
    outs = []
    for hint, mx in [([1, 1, 1], 32), ([32, 32, 32], 32), ([7, 2, 3], 8), ([128, 128, 128], 128), ([40, 3, 17], 64)]:
        s = torch.tensor(hint, dtype=torch.int32).cuda()
        out = run(q, kc, vc, indptr, slots, s, mx)
        assert_close_to_oracle(out, ref, f"hint {hint}")
        outs.append(out.float())
    for o in outs[1:]:
        assert (o - outs[0]).abs().max() <= 1.6e-2  # bf16 rounding of differently ordered fp32 sums


def test_empty_sequence_gives_zeros_and_neighbours_are_untouched():
    q, kc, vc, _, slots, _ = make_inputs([300, 40], 2, 8, seed=5)
    indptr = torch.tensor([0, 300, 300, 340], dtype=torch.int32).cuda()
    q = torch.cat([q[:1], q[:1], q[1:]])
    splits = torch.tensor([3, 1, 1], dtype=torch.int32).cuda()
    out = run(q, kc, vc, indptr, slots, splits)
    assert torch.count_nonzero(out[1]) == 0
    ref = O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, 1 / math.sqrt(128))
    assert_close_to_oracle(out, ref, "empty middle sequence")


def test_shared_prefix_slots_between_sequences():
    # radix-cache reuse: two sequences list the same slot ids for their common prefix
    g = torch.Generator().manual_seed(9)
    hkv, hq, d = 2, 8, 128
    kc = torch.randn(600, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(600, hkv, d, generator=g).bfloat16().cuda()
    perm = torch.randperm(600, generator=g).int()
    shared, a, b = perm[:200], perm[200:300], perm[300:450]
    slots = torch.cat([shared, a, shared, b]).cuda()
    indptr = torch.tensor([0, 300, 650], dtype=torch.int32).cuda()
    q = torch.randn(2, hq, d, generator=g).bfloat16().cuda()
    splits = torch.tensor([3, 3], dtype=torch.int32).cuda()
    ref = O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, 1 / math.sqrt(d))
    assert_close_to_oracle(run(q, kc, vc, indptr, slots, splits), ref, "shared prefix")


def test_float16():
    args = make_inputs([700, 33], 2, 8, seed=21, dtype=torch.float16)
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128))
    assert_close_to_oracle(run(*args), ref, "f16")


def test_out_of_range_slot_is_reported_not_dereferenced():
    from mini_sglang_mlx_b200.kernel import device_status
    q, kc, vc, indptr, slots, splits = make_inputs([100], 2, 4, seed=2)
    device_status()
    bad = slots.clone()
    bad[17] = kc.shape[0] + 5
    out = run(q, kc, vc, indptr, bad, splits)
    assert torch.isfinite(out.float()).all()
    assert device_status() == 2
    assert device_status() == 0


def test_cfg1_full_size():
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg1_decode()
    out = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, w.num_kv_splits, w.max_kv_splits)
    ref = O.paged_decode_attention_oracle(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, w.sm_scale)
    assert_close_to_oracle(out, ref, "cfg1")


def test_cfg5a_reduced_and_properties():
    """Long-context decode at 1/8 of the batch (full lengths): a subsample of sequences against the
    oracle, then split-count invariance over all of them."""
    from mini_sglang_mlx_b200 import synthetic as S
    from mini_sglang_mlx_b200.attention import compute_num_kv_splits
    w = S.cfg5a_decode(batch=32)
    out = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, w.num_kv_splits, w.max_kv_splits)
    order = sorted(range(w.batch), key=lambda b: w.kv_lens[b])
    pick = [order[0], order[len(order) // 2], order[-1]]
    ref = O.paged_decode_attention_oracle(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices,
                                          w.sm_scale, seqs=pick)
    assert_close_to_oracle(out[pick], ref[pick], "cfg5a subsample")
    tuned = torch.tensor(compute_num_kv_splits(w.kv_lens, w.hkv), dtype=torch.int32).cuda()
    out2 = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, tuned, 32)
    assert (out.float() - out2.float()).abs().max() <= 1.6e-2


def test_cfg5a_full_size_properties():
    """The long-context decode batch at its full size (256 sequences, 38 GB of K/V), checked through
    properties that need no full-size oracle: the result does not depend on the split counts beyond
    rounding, doubling V doubles the output bit for bit (a power-of-two factor commutes with every
    rounding on the path), and 16 of the 256 sequences (evenly spaced in the order of their lengths,
    shortest and longest included) agree with the oracle."""
    from mini_sglang_mlx_b200 import synthetic as S
    from mini_sglang_mlx_b200.attention import compute_num_kv_splits
    w = S.cfg5a_decode()
    tuned = torch.tensor(compute_num_kv_splits(w.kv_lens, w.hkv), dtype=torch.int32).cuda()
    out = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, tuned, w.max_kv_splits)
    assert torch.isfinite(out.float()).all()
    ref_splits = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, w.num_kv_splits, w.max_kv_splits)
    assert (out.float() - ref_splits.float()).abs().max() <= 1.6e-2
    order = sorted(range(w.batch), key=lambda b: w.kv_lens[b])
    pick = sorted({order[round(i * (len(order) - 1) / 15)] for i in range(16)})
    ref = O.paged_decode_attention_oracle(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices,
                                          w.sm_scale, seqs=pick)
    assert_close_to_oracle(out[pick], ref[pick], "cfg5a full size, subsample")
    w.v_cache.mul_(2)
    doubled = run(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, tuned, w.max_kv_splits)
    assert torch.equal(doubled, out * 2)


def test_more_sequence_head_pairs_than_the_header_has_counters():
    """batch * Hq beyond the 16384 arrival counters of the workspace header: the op keeps the
    counters in a region of its own and clears it on every call."""
    kv_lens = [130 + (i % 7) * 64 for i in range(2100)]
    args = make_inputs(kv_lens, 2, 8, seed=12)
    splits = torch.full((len(kv_lens),), 3, dtype=torch.int32).cuda()
    for _ in range(2):
        out = run(*args[:5], splits)
    pick = [0, 1000, 2099]
    ref = O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128), seqs=pick)
    assert_close_to_oracle(out[pick], ref[pick], "decode, 2100 sequences")
