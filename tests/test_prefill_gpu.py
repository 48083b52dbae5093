"""Paged prefill / verify / block attention on the GPU against the oracle and
the reference's analytic mask cases."""
import math

import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle, build_kat_inputs, load_mask_kats

pytestmark = pytest.mark.gpu

KATS = load_mask_kats()
HEAD_CONFIGS = [(2, 16), (4, 16), (4, 24), (2, 32), (8, 32), (1, 1)]  # (Hkv, Hq)


def make_inputs(q_lens, prefix_lens, hkv, hq, *, seed=0, d=128, permute=True, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    kv_lens = [a + b for a, b in zip(q_lens, prefix_lens)]
    total = sum(kv_lens)
    S = total + 9
    kc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    q = torch.randn(sum(q_lens), hq, d, generator=g).to(dtype).cuda()
    slots = (torch.randperm(S, generator=g)[:total] if permute else torch.arange(total)).int().cuda()
    return dict(q=q, k_cache=kc, v_cache=vc, qo_indptr=torch.from_numpy(O.build_indptr(q_lens)).cuda(),
                kv_indptr=torch.from_numpy(O.build_indptr(kv_lens)).cuda(), kv_indices=slots,
                prefix_lens=torch.tensor(prefix_lens, dtype=torch.int32).cuda(),
                max_len_extend=max(q_lens))


def run(d, cross=False, window=0):
    from mini_sglang_mlx_b200 import paged_prefill_attention
    out = paged_prefill_attention(d["q"], d["k_cache"], d["v_cache"], d["qo_indptr"], d["kv_indptr"],
                                  d["kv_indices"], d["prefix_lens"], 1 / math.sqrt(d["q"].shape[-1]),
                                  d["max_len_extend"], is_cross_attention=cross,
                                  sliding_window_size=window)
    torch.cuda.synchronize()
    return out


def oracle(d, cross=False, window=0, **kw):
    return O.paged_prefill_attention_oracle(d["q"], d["k_cache"], d["v_cache"], d["qo_indptr"],
                                            d["kv_indptr"], d["kv_indices"], d["prefix_lens"],
                                            1 / math.sqrt(d["q"].shape[-1]), is_cross_attention=cross,
                                            sliding_window_size=window, **kw)


@pytest.mark.parametrize("case", KATS, ids=[c["name"] for c in KATS])
def test_reference_mask_known_answers(case):
    from mini_sglang_mlx_b200 import paged_prefill_attention, store_kv_cache
    d = build_kat_inputs(case, device="cuda")
    v_cache = torch.zeros_like(d["k_cache"])
    if case["slots"] is None:
        v_cache[: d["kv_len"]] = d["v_rows"]
    else:
        store_kv_cache(d["k_cache"], v_cache, d["kv_indices"], torch.zeros_like(d["v_rows"]), d["v_rows"])
    out = paged_prefill_attention(d["q"], d["k_cache"], v_cache, d["qo_indptr"], d["kv_indptr"],
                                  d["kv_indices"], d["prefix_lens"], sm_scale=d["sm_scale"],
                                  max_len_extend=case["q_len"],
                                  is_cross_attention=case["is_cross_attention"],
                                  sliding_window_size=case["sliding_window_size"])
    actual = out.float().cpu().numpy()[:, 0, : d["kv_len"]]
    np.testing.assert_allclose(actual, np.asarray(case["expected_weights"], dtype=np.float32),
                               rtol=case["rtol"], atol=case["atol"])


@pytest.mark.parametrize("hkv,hq", HEAD_CONFIGS)
@pytest.mark.parametrize("q_len", [1, 237, 512, 809, 1024, 2048])
def test_pure_prefill(hkv, hq, q_len):
    d = make_inputs([q_len], [0], hkv, hq, seed=q_len)
    assert_close_to_oracle(run(d), oracle(d), f"prefill q={q_len} Hkv={hkv} Hq={hq}")


@pytest.mark.parametrize("q_len", [3333, 4096])
def test_pure_prefill_long(q_len):
    d = make_inputs([q_len], [0], 2, 8, seed=q_len)
    assert_close_to_oracle(run(d), oracle(d), f"prefill q={q_len}")


@pytest.mark.parametrize("hkv,hq", HEAD_CONFIGS[:5])
@pytest.mark.parametrize("q_len,prefix", [(237, 100), (512, 256), (1024, 512), (2048, 1024)])
def test_prefix_extend(hkv, hq, q_len, prefix):
    d = make_inputs([q_len], [prefix], hkv, hq, seed=prefix)
    assert_close_to_oracle(run(d), oracle(d), f"extend q={q_len} prefix={prefix}")


RAGGED = [([1, 237], [0, 0]), ([512, 1024], [0, 0]), ([237, 809, 1024], [0, 100, 512]),
          ([1, 512, 2048, 4096], [0, 0, 0, 0]), ([128, 256, 512, 1024], [64, 128, 256, 512])]


@pytest.mark.parametrize("hkv,hq", [(2, 16), (4, 24), (8, 32)])
@pytest.mark.parametrize("q_lens,prefixes", RAGGED, ids=[str(r[0]) for r in RAGGED])
def test_ragged_batch(hkv, hq, q_lens, prefixes):
    d = make_inputs(q_lens, prefixes, hkv, hq, seed=len(q_lens))
    assert_close_to_oracle(run(d), oracle(d), f"ragged {q_lens} {prefixes}")


@pytest.mark.parametrize("cross,window", [(False, 0), (True, 0), (False, 64), (True, 64), (False, 1),
                                          (False, 1000), (True, 1), (False, 129), (True, 4096)])
@pytest.mark.parametrize("q_lens,prefixes", [([16, 8, 1], [500, 77, 130]), ([200, 65], [0, 300])])
def test_mask_modes(cross, window, q_lens, prefixes):
    d = make_inputs(q_lens, prefixes, 2, 8, seed=window + 13 * cross)
    assert_close_to_oracle(run(d, cross, window), oracle(d, cross, window),
                           f"mask cross={cross} W={window} {q_lens}")


def test_sequence_without_query_tokens_in_a_ragged_batch():
    d = make_inputs([5, 0, 9], [10, 20, 0], 2, 8, seed=4)
    d["max_len_extend"] = 9
    assert_close_to_oracle(run(d), oracle(d), "Tq=0 in the middle")


def test_one_query_token_equals_the_decode_op():
    from mini_sglang_mlx_b200 import paged_decode_attention
    lens = [1, 77, 1300]
    d = make_inputs([1, 1, 1], [l - 1 for l in lens], 4, 16, seed=8)
    out_p = run(d)
    splits = torch.from_numpy(O.compute_num_kv_splits(lens)).cuda()
    out_d = paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["kv_indptr"], d["kv_indices"],
                                   splits, 1 / math.sqrt(128), 32)
    assert (out_p.float() - out_d.float()).abs().max() <= 1.6e-2
    assert_close_to_oracle(out_p, oracle(d), "Tq=1 via prefill")


def test_verify_shape_with_kv_split():
    # few query tiles and long prefixes: the kv-split path with its merge pass
    d = make_inputs([8] * 6, [5000, 1024, 33, 9000, 2047, 700], 4, 32, seed=31)
    assert_close_to_oracle(run(d), oracle(d), "verify K+1=8")


def test_bidirectional_block_with_window_and_kv_split():
    d = make_inputs([16] * 4, [8176, 4000, 100, 5000], 8, 32, seed=32)
    for cross in (False, True):
        assert_close_to_oracle(run(d, cross, 4096), oracle(d, cross, 4096), f"block cross={cross}")


def test_float16():
    d = make_inputs([100, 7], [30, 900], 2, 8, seed=6, dtype=torch.float16)
    assert_close_to_oracle(run(d), oracle(d), "f16")


def _run_workload(w):
    from mini_sglang_mlx_b200 import paged_prefill_attention
    out = paged_prefill_attention(w.q, w.k_cache, w.v_cache, w.qo_indptr, w.kv_indptr, w.kv_indices,
                                  w.prefix_lens, w.sm_scale, w.max_len_extend,
                                  is_cross_attention=w.is_cross_attention,
                                  sliding_window_size=w.sliding_window_size)
    torch.cuda.synchronize()
    return out


def _oracle_workload(w, **kw):
    return O.paged_prefill_attention_oracle(w.q, w.k_cache, w.v_cache, w.qo_indptr, w.kv_indptr,
                                            w.kv_indices, w.prefix_lens, w.sm_scale,
                                            is_cross_attention=w.is_cross_attention,
                                            sliding_window_size=w.sliding_window_size, **kw)


def test_cfg2_full_size():
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg2_prefill()
    assert_close_to_oracle(_run_workload(w), _oracle_workload(w), "cfg2")


@pytest.mark.parametrize("cross", [False, True])
def test_cfg3_full_size(cross):
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg3_window_block(cross=cross)
    assert_close_to_oracle(_run_workload(w), _oracle_workload(w), f"cfg3 cross={cross}")


def test_cfg4_full_size():
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg4_verify()
    assert_close_to_oracle(_run_workload(w), _oracle_workload(w), "cfg4")


@pytest.mark.parametrize("chunk,prefix", [(128, 1024), (128, 32768), (1024, 4096), (4096, 1024)])
def test_cfg5b_points(chunk, prefix):
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg5b_prefill_point(chunk, prefix)
    assert_close_to_oracle(_run_workload(w), _oracle_workload(w), f"cfg5b {chunk}x{prefix}")


# ---------------------------------------------------------------- head_dim 256
# (the reference's prefill op accepts 128 and 256: csrc/paged_prefill_attention.cpp:53-56)
@pytest.mark.parametrize("hkv,hq", [(2, 8), (4, 16), (1, 1), (2, 16)])
@pytest.mark.parametrize("q_lens,prefixes", [([1], [0]), ([237], [0]), ([64], [700]), ([300, 17, 128], [100, 2000, 0]),
                                            ([1024], [512])])
def test_head_dim_256(hkv, hq, q_lens, prefixes):
    d = make_inputs(q_lens, prefixes, hkv, hq, seed=sum(q_lens) + hq, d=256)
    assert_close_to_oracle(run(d), oracle(d), f"D=256 q{q_lens} prefix{prefixes} Hkv{hkv}/Hq{hq}")


@pytest.mark.parametrize("cross,window", [(False, 0), (True, 0), (False, 64), (True, 64), (False, 1)])
def test_head_dim_256_mask_modes(cross, window):
    d = make_inputs([16, 8, 1, 200], [500, 77, 130, 0], 2, 8, seed=3, d=256)
    assert_close_to_oracle(run(d, cross, window), oracle(d, cross, window), f"D=256 cross={cross} W={window}")


def test_head_dim_256_long_keys_take_the_split_path_and_f16():
    d = make_inputs([8, 8], [9000, 3000], 2, 16, seed=5, d=256)          # few query tiles: key range is split
    assert_close_to_oracle(run(d), oracle(d), "D=256 verify shape")
    d = make_inputs([130], [260], 4, 16, seed=6, d=256, dtype=torch.float16)
    assert_close_to_oracle(run(d), oracle(d), "D=256 f16")


def test_head_dim_256_one_query_token_equals_the_decode_op():
    from mini_sglang_mlx_b200 import paged_decode_attention
    d = make_inputs([1, 1, 1], [1500, 63, 4097], 4, 16, seed=8, d=256)
    out_p = run(d)
    splits = torch.tensor([4, 1, 8], dtype=torch.int32).cuda()
    out_d = paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["kv_indptr"], d["kv_indices"], splits,
                                   1 / math.sqrt(256), 8)
    assert (out_p.float() - out_d.float()).abs().max().item() <= 2e-2


def test_cfg5b_largest_point_properties():
    """Chunk 4096 over a cached prefix of 32768 tokens (the largest grid point): the first and the
    last 64 query tokens against the oracle (as 64-token chunks behind a longer prefix: the same
    rows of the same problem), and doubling V doubles the output bit for bit."""
    from mini_sglang_mlx_b200 import synthetic as S
    w = S.cfg5b_prefill_point(4096, 32768)
    out = _run_workload(w)
    assert torch.isfinite(out.float()).all()
    n = 64
    for first in (0, 4096 - n):
        qo = torch.tensor([0, n], dtype=torch.int32, device=out.device)
        kvp = torch.tensor([0, 32768 + first + n], dtype=torch.int32, device=out.device)
        pre = torch.tensor([32768 + first], dtype=torch.int32, device=out.device)
        ref = O.paged_prefill_attention_oracle(w.q[first:first + n], w.k_cache, w.v_cache, qo, kvp,
                                               w.kv_indices[: 32768 + first + n], pre, w.sm_scale)
        assert_close_to_oracle(out[first:first + n], ref, f"cfg5b 4096x32768 rows {first}..")
    w.v_cache.mul_(2)
    assert torch.equal(_run_workload(w), out * 2)


@pytest.mark.parametrize("hkv,hq,kv_hi", [(2, 8, 700), (1, 4, 5000)], ids=["unsplit", "split"])
def test_batches_of_more_than_128_sequences(hkv, hq, kv_hi):
    """Above 128 sequences the CTAs find their work item by a running scan in the natural order
    instead of the sorted search; (1, 4): few enough query tiles for the key range to be split
    (two launches or arrival counters), (2, 8): unsplit.  Ragged lengths, some sequences without
    query tokens."""
    rng = np.random.default_rng(11)
    batch = 140
    q_lens = rng.integers(0, 9, size=batch).tolist()
    q_lens[3] = 8
    prefixes = rng.integers(0, kv_hi, size=batch).tolist()
    d = make_inputs(q_lens, prefixes, hkv, hq, seed=41)
    assert_close_to_oracle(run(d), oracle(d), f"batch of {batch}, kv up to {kv_hi}")
