"""Page-granular index entries (one id per page of page_size tokens) on the GPU.

The reference has one token per page (mini_sglang_mlx/engine/engine.py:103) and per-token
``kv_indices``; these entries take (page_indptr, page_indices, kv_lens) instead.  With a page
size that is a multiple of 16 the kernels fetch K/V as TMA boxes straight from the page ids;
other page sizes build per-token ids on the device first.  Checked against the fp32 oracle
(every benchmark configuration, ragged and boundary lengths, all mask modes, f16, head_dim 256)
and against the per-token ops on the same pool.
"""
import math

import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu


def make_pool(kv_lens, page_size, hkv, *, seed=0, d=128, spare_pages=5, dtype=torch.bfloat16):
    """Pages drawn by random permutation; returns caches, page CSR and the per-token slot ids."""
    g = torch.Generator().manual_seed(seed)
    need = [(l + page_size - 1) // page_size for l in kv_lens]
    num_pages = sum(need) + spare_pages
    perm = torch.randperm(num_pages, generator=g).int()
    page_indptr = torch.tensor([0] + list(torch.tensor(need).cumsum(0).tolist()), dtype=torch.int32)
    page_indices = perm[: sum(need)].contiguous()
    slots = []
    for b, l in enumerate(kv_lens):
        t = torch.arange(l)
        pages = page_indices[page_indptr[b]: page_indptr[b + 1]].long()
        slots.append((pages[t // page_size] * page_size + t % page_size).int())
    slots = torch.cat(slots) if slots else torch.zeros(0, dtype=torch.int32)
    S = num_pages * page_size
    kc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(S, hkv, d, generator=g).to(dtype).cuda()
    return kc, vc, page_indptr.cuda(), page_indices.cuda(), slots.cuda()


@pytest.mark.parametrize("page_size", [1, 16, 32, 48, 64])
@pytest.mark.parametrize("kv_lens", [[1], [237, 809], [16, 32, 48], [0, 5, 0, 4097], [2048] * 3 + [1],
                                     [15, 17, 63, 65, 1023, 1025]], ids=str)
def test_decode_matches_the_per_token_op_and_the_oracle(page_size, kv_lens):
    from mini_sglang_mlx_b200 import paged_decode_attention, paged_decode_attention_p16
    hkv, hq, d = 4, 16, 128
    kc, vc, pip, pidx, slots = make_pool(kv_lens, page_size, hkv, seed=len(kv_lens) + page_size)
    g = torch.Generator().manual_seed(7)
    q = torch.randn(len(kv_lens), hq, d, generator=g).bfloat16().cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
    scale = 1 / math.sqrt(d)
    out = paged_decode_attention_p16(q, kc, vc, pip, pidx, lens, splits, scale, 32, page_size=page_size)
    same = paged_decode_attention(q, kc, vc, indptr, slots, splits, scale, 32)
    torch.cuda.synchronize()
    assert torch.equal(out, same)
    ref = O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, scale)
    assert_close_to_oracle(out, ref, f"decode p{page_size} {kv_lens}")


@pytest.mark.parametrize("page_size", [1, 16, 32, 48])
@pytest.mark.parametrize("case", [
    dict(q_lens=[5, 17], prefix=[0, 40]),
    dict(q_lens=[1, 16, 15, 17], prefix=[0, 0, 1, 47]),
    dict(q_lens=[300, 64], prefix=[129, 8000]),
    dict(q_lens=[700], prefix=[0], window=100),
    dict(q_lens=[16, 16], prefix=[8176, 5000], window=4096, cross=True),
    dict(q_lens=[512], prefix=[1000]),
    dict(q_lens=[16] * 4, prefix=[3000, 100, 0, 2047], window=1024),
    dict(q_lens=[8, 8], prefix=[4000, 6000]),                       # short block: key range is split
    dict(q_lens=[33, 1], prefix=[64, 64], cross=True),
    dict(q_lens=[0, 9, 0, 4], prefix=[50, 0, 0, 700]),              # sequences without query tokens / keys
], ids=str)
def test_prefill_matches_the_per_token_op_and_the_oracle(page_size, case):
    from mini_sglang_mlx_b200 import paged_prefill_attention, paged_prefill_attention_p16
    hkv, hq, d = 2, 8, 128
    q_lens, prefix = case["q_lens"], case["prefix"]
    window, cross = case.get("window", 0), case.get("cross", False)
    kv_lens = [p + t for p, t in zip(prefix, q_lens)]
    kc, vc, pip, pidx, slots = make_pool(kv_lens, page_size, hkv, seed=sum(kv_lens) % 97)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(sum(q_lens), hq, d, generator=g).bfloat16().cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    pre = torch.tensor(prefix, dtype=torch.int32).cuda()
    qo = torch.from_numpy(O.build_indptr(q_lens)).cuda()
    kvp = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    scale = 1 / math.sqrt(d)
    kw = dict(is_cross_attention=cross, sliding_window_size=window)
    out = paged_prefill_attention_p16(q, kc, vc, qo, pip, pidx, lens, pre, scale, max(q_lens),
                                      page_size=page_size, **kw)
    same = paged_prefill_attention(q, kc, vc, qo, kvp, slots, pre, scale, max(q_lens), **kw)
    torch.cuda.synchronize()
    # the same kernels on the same slot ids; only the key-range split may differ (it is sized
    # from total_pages * page_size here, from the exact token count there)
    assert (out.float() - same.float()).abs().max().item() <= 2e-2
    ref = O.paged_prefill_attention_oracle(q, kc, vc, qo, kvp, slots, pre, scale, **kw)
    assert_close_to_oracle(out, ref, f"prefill p{page_size} {case}")


def test_a_length_beyond_the_pages_of_a_sequence_is_reported_and_clamped():
    from mini_sglang_mlx_b200 import paged_decode_attention_p16
    from mini_sglang_mlx_b200.kernel import device_status
    hkv, hq, d, ps = 2, 4, 128, 16
    kv_lens = [40, 20]
    kc, vc, pip, pidx, _ = make_pool(kv_lens, ps, hkv, seed=3)
    q = torch.randn(2, hq, d).bfloat16().cuda()
    splits = torch.ones(2, dtype=torch.int32).cuda()
    device_status()
    bad = torch.tensor([40, 33], dtype=torch.int32).cuda()       # sequence 1 owns 2 pages = 32 tokens
    out = paged_decode_attention_p16(q, kc, vc, pip, pidx, bad, splits, 0.1, 32, page_size=ps)
    assert device_status() == 2
    clamped = torch.tensor([40, 32], dtype=torch.int32).cuda()
    ok = paged_decode_attention_p16(q, kc, vc, pip, pidx, clamped, splits, 0.1, 32, page_size=ps)
    assert device_status() == 0
    assert torch.equal(out, ok)


def test_workspace_size_is_checked_through_the_c_abi():
    from mini_sglang_mlx_b200 import _lib
    lib = _lib.lib()
    idx = lib.msgl_page_index_workspace_bytes(3, 100, 16)
    assert idx >= (3 + 1 + 1600) * 4 and idx % 256 == 0
    q = torch.zeros(3, 4, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1600, 2, 128, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(101, dtype=torch.int32, device="cuda")
    ws = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    rc = lib.msgl_paged_decode_attention_p16(
        q.data_ptr(), kc.data_ptr(), kc.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
        None, q.data_ptr(), ws.data_ptr(), ws.numel(), 3, 4, 2, 128, 1600, _lib.DTYPE_BF16, 0.1, 32, 16,
        100, 0)
    assert rc != 0 and "workspace too small" in lib.msgl_last_error_string().decode()


# ---------------------------------------------------------------- the benchmark configurations
def _oracle_for(w, seqs=None):
    if w.kind == "decode":
        kw = {} if seqs is None else {"seqs": seqs}
        return O.paged_decode_attention_oracle(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices,
                                               w.sm_scale, **kw)
    return O.paged_prefill_attention_oracle(w.q, w.k_cache, w.v_cache, w.qo_indptr, w.kv_indptr,
                                            w.kv_indices, w.prefix_lens, w.sm_scale,
                                            is_cross_attention=w.is_cross_attention,
                                            sliding_window_size=w.sliding_window_size)


def _run_paged(w, splits=None):
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, paged_prefill_attention_p16
    pip, pidx, lens = w.page_csr()
    if w.kind == "decode":
        out = paged_decode_attention_p16(w.q, w.k_cache, w.v_cache, pip, pidx, lens,
                                         w.num_kv_splits if splits is None else splits, w.sm_scale,
                                         w.max_kv_splits)
    else:
        out = paged_prefill_attention_p16(w.q, w.k_cache, w.v_cache, w.qo_indptr, pip, pidx, lens,
                                          w.prefix_lens, w.sm_scale, w.max_len_extend,
                                          is_cross_attention=w.is_cross_attention,
                                          sliding_window_size=w.sliding_window_size)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3", "cfg3_cross", "cfg4", "cfg5b_128_1024",
                                  "cfg5b_128_32768", "cfg5b_1024_4096", "cfg5b_4096_1024"])
def test_benchmark_configurations_against_the_oracle(name):
    from mini_sglang_mlx_b200 import synthetic as S
    from mini_sglang_mlx_b200.kernel import device_status
    w = {"cfg1": S.cfg1_decode, "cfg2": S.cfg2_prefill, "cfg3": S.cfg3_window_block,
         "cfg3_cross": lambda: S.cfg3_window_block(cross=True), "cfg4": S.cfg4_verify}.get(name)
    w = w() if w else S.cfg5b_prefill_point(*map(int, name.split("_")[1:]))
    device_status()
    out = _run_paged(w)
    assert device_status() == 0
    assert_close_to_oracle(out, _oracle_for(w), f"{name} through the page-granular entry")


def test_cfg5a_reduced_against_the_oracle_and_the_per_token_op():
    from mini_sglang_mlx_b200 import paged_decode_attention, synthetic as S
    w = S.cfg5a_decode(batch=32)
    out = _run_paged(w)
    order = sorted(range(w.batch), key=lambda b: w.kv_lens[b])
    pick = [order[0], order[len(order) // 2], order[-1]]
    ref = _oracle_for(w, seqs=pick)
    assert_close_to_oracle(out[pick], ref[pick], "cfg5a subsample, page-granular")
    same = paged_decode_attention(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, w.num_kv_splits,
                                  w.sm_scale, w.max_kv_splits)
    assert (out.float() - same.float()).abs().max().item() <= 1.6e-2


def test_cfg5a_full_size_properties():
    """The long-context decode batch at full size (38 GB of K/V) through the page-granular entry:
    split-count invariance, exact doubling with V, 16 of the 256 sequences (evenly spaced in the
    order of their lengths) against the oracle, and all 256 against the per-token operator."""
    from mini_sglang_mlx_b200 import paged_decode_attention, synthetic as S
    from mini_sglang_mlx_b200.attention import compute_num_kv_splits
    w = S.cfg5a_decode()
    tuned = torch.tensor(compute_num_kv_splits(w.kv_lens, w.hkv), dtype=torch.int32).cuda()
    out = _run_paged(w, tuned)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - _run_paged(w).float()).abs().max() <= 1.6e-2
    per_token = paged_decode_attention(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, tuned,
                                       w.sm_scale, w.max_kv_splits)
    assert (out.float() - per_token.float()).abs().max() <= 1.6e-2
    del per_token
    order = sorted(range(w.batch), key=lambda b: w.kv_lens[b])
    pick = sorted({order[round(i * (len(order) - 1) / 15)] for i in range(16)})
    ref = _oracle_for(w, seqs=pick)
    assert_close_to_oracle(out[pick], ref[pick], "cfg5a full size, page-granular, subsample")
    w.v_cache.mul_(2)
    assert torch.equal(_run_paged(w, tuned), out * 2)


# ---------------------------------------------------------------- edges of the TMA path
def test_rows_past_a_sequence_end_are_never_used():
    """The last page of a sequence is ragged; the pool rows behind its last token (and every
    unowned page) hold NaN here.  Nothing of them may reach the output."""
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, paged_prefill_attention_p16
    hkv, hq, d, ps = 2, 8, 128, 16
    kv_lens = [1, 17, 130, 1000, 2049]
    q_lens = [1, 9, 64, 8, 300]
    kc, vc, pip, pidx, slots = make_pool(kv_lens, ps, hkv, seed=21)
    used = torch.zeros(kc.shape[0], dtype=torch.bool, device="cuda")
    used[slots.long()] = True
    kc[~used] = float("nan")
    vc[~used] = float("nan")
    lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    scale = 1 / math.sqrt(d)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(len(kv_lens), hq, d, generator=g).bfloat16().cuda()
    splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
    out = paged_decode_attention_p16(q, kc, vc, pip, pidx, lens, splits, scale, 32, page_size=ps)
    ref = O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, scale)
    assert_close_to_oracle(out, ref, "decode over a pool with NaN outside the sequences")
    qp = torch.randn(sum(q_lens), hq, d, generator=g).bfloat16().cuda()
    qo = torch.from_numpy(O.build_indptr(q_lens)).cuda()
    pre = torch.tensor([l - t for l, t in zip(kv_lens, q_lens)], dtype=torch.int32).cuda()
    for cross, window in ((False, 0), (True, 0), (False, 50)):
        outp = paged_prefill_attention_p16(qp, kc, vc, qo, pip, pidx, lens, pre, scale, max(q_lens),
                                           page_size=ps, is_cross_attention=cross,
                                           sliding_window_size=window)
        refp = O.paged_prefill_attention_oracle(qp, kc, vc, qo, indptr, slots, pre, scale,
                                                is_cross_attention=cross, sliding_window_size=window)
        assert_close_to_oracle(outp, refp, f"prefill over a pool with NaN outside (cross={cross}, W={window})")


def test_a_page_outside_the_pool_is_reported_and_read_as_zeros():
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, paged_prefill_attention_p16
    from mini_sglang_mlx_b200.kernel import device_status
    hkv, hq, d, ps = 2, 4, 128, 16
    kv_lens = [100, 40]
    kc, vc, pip, pidx, _ = make_pool(kv_lens, ps, hkv, seed=4)
    bad = pidx.clone()
    bad[2] = kc.shape[0] // ps + 3            # a page id past the pool
    bad[8] = -2
    lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    q = torch.randn(2, hq, d).bfloat16().cuda()
    splits = torch.ones(2, dtype=torch.int32).cuda()
    device_status()
    out = paged_decode_attention_p16(q, kc, vc, pip, bad, lens, splits, 0.1, 32, page_size=ps)
    assert device_status() == 2
    assert torch.isfinite(out.float()).all()
    qo = torch.tensor([0, 1, 2], dtype=torch.int32).cuda()
    pre = torch.tensor([99, 39], dtype=torch.int32).cuda()
    outp = paged_prefill_attention_p16(q, kc, vc, qo, pip, bad, lens, pre, 0.1, 1, page_size=ps)
    assert device_status() == 2
    assert torch.isfinite(outp.float()).all()


def test_shared_prefix_pages_and_float16_and_head_dim_256():
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, paged_prefill_attention_p16
    ps = 16
    for d, dtype, hkv, hq in ((128, torch.float16, 2, 8), (256, torch.bfloat16, 2, 8), (256, torch.float16, 1, 4)):
        kv_lens = [700, 333, 64]
        q_lens = [60, 13, 64]
        kc, vc, pip, pidx, slots = make_pool(kv_lens, ps, hkv, seed=d + hq, d=d, dtype=dtype)
        # sequence 1 re-uses the first 20 pages of sequence 0 (a shared cached prefix)
        pidx = pidx.clone()
        start0, start1 = int(pip[0]), int(pip[1])
        pidx[start1:start1 + 20] = pidx[start0:start0 + 20]
        slots = slots.clone()
        o0, o1 = 0, kv_lens[0]
        slots[o1:o1 + 320] = slots[o0:o0 + 320]
        lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
        indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
        scale = 1 / math.sqrt(d)
        g = torch.Generator().manual_seed(d)
        q = torch.randn(len(kv_lens), hq, d, generator=g).to(dtype).cuda()
        splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
        out = paged_decode_attention_p16(q, kc, vc, pip, pidx, lens, splits, scale, 32, page_size=ps)
        assert_close_to_oracle(out, O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, scale),
                               f"decode D={d} {dtype}")
        qp = torch.randn(sum(q_lens), hq, d, generator=g).to(dtype).cuda()
        qo = torch.from_numpy(O.build_indptr(q_lens)).cuda()
        pre = torch.tensor([l - t for l, t in zip(kv_lens, q_lens)], dtype=torch.int32).cuda()
        outp = paged_prefill_attention_p16(qp, kc, vc, qo, pip, pidx, lens, pre, scale, max(q_lens),
                                           page_size=ps)
        refp = O.paged_prefill_attention_oracle(qp, kc, vc, qo, indptr, slots, pre, scale)
        assert_close_to_oracle(outp, refp, f"prefill D={d} {dtype}")


def test_mask_known_answers_through_the_page_entry():
    """The reference's analytic mask cases (identity slots) with the pool seen as 16-token pages."""
    from mini_sglang_mlx_b200 import paged_prefill_attention_p16, store_kv_cache
    from tests.helpers import build_kat_inputs, load_mask_kats
    ps = 16
    for case in load_mask_kats():
        if case["slots"] is not None:
            continue                      # permuted per-token slots have no page-granular form
        d = build_kat_inputs(case, device="cuda")
        npages = (d["kv_len"] + ps - 1) // ps
        kc = torch.zeros(npages * ps, 1, case["head_dim"], dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        store_kv_cache(kc, vc, d["kv_indices"], torch.zeros_like(d["v_rows"]), d["v_rows"])
        pip = torch.tensor([0, npages], dtype=torch.int32).cuda()
        pidx = torch.arange(npages, dtype=torch.int32).cuda()
        lens = torch.tensor([d["kv_len"]], dtype=torch.int32).cuda()
        out = paged_prefill_attention_p16(d["q"], kc, vc, d["qo_indptr"], pip, pidx, lens, d["prefix_lens"],
                                          d["sm_scale"], case["q_len"], page_size=ps,
                                          is_cross_attention=case["is_cross_attention"],
                                          sliding_window_size=case["sliding_window_size"])
        want = torch.tensor(case["expected_weights"], dtype=torch.float32)
        got = out.float().cpu()[:, 0, : d["kv_len"]]
        assert torch.allclose(got, want, rtol=case["rtol"], atol=case["atol"]), case["name"]


def test_prefill_batches_of_more_than_128_sequences():
    """The work-item scan of large batches (natural order, no sorting) on the page-granular path,
    unsplit and with the key range split."""
    import numpy as np
    from mini_sglang_mlx_b200 import synthetic as S
    rng = np.random.default_rng(12)
    for hkv, hq, kv_hi in ((2, 8, 700), (1, 4, 5000)):
        q_lens = rng.integers(1, 9, size=140).tolist()
        prefixes = rng.integers(0, kv_hi, size=140).tolist()
        pages = sum((a + b + 15) // 16 for a, b in zip(q_lens, prefixes))
        w = S.make_prefill("large_batch", hq=hq, hkv=hkv, q_lens=q_lens, prefix_lens=prefixes,
                           num_pages=pages + 32, seed=77 + hkv, device="cuda")
        assert_close_to_oracle(_run_paged(w), _oracle_for(w), f"140 sequences, kv up to {kv_hi}")


@pytest.mark.parametrize("hkv,hq", [(4, 24), (2, 24), (1, 1), (2, 32), (3, 15)], ids=str)
def test_prefill_head_ratios(hkv, hq):
    """Query heads per KV head that divide 128 (the query tile arrives as TMA boxes) and that do
    not (6, 12, 5: 16-byte copies by the producer warps), short and long query blocks."""
    from mini_sglang_mlx_b200 import synthetic as S
    for q_lens, prefixes in (([8, 3], [700, 2500]), ([300, 77], [100, 0])):
        pages = sum((a + b + 15) // 16 for a, b in zip(q_lens, prefixes))
        w = S.make_prefill("heads", hq=hq, hkv=hkv, q_lens=q_lens, prefix_lens=prefixes,
                           num_pages=pages + 8, seed=5 + hq, device="cuda")
        assert_close_to_oracle(_run_paged(w), _oracle_for(w), f"heads ({hkv}, {hq}) q {q_lens}")


@pytest.mark.parametrize("hkv,hq", [(4, 24), (1, 1), (2, 32), (3, 15)], ids=str)
def test_decode_head_ratios(hkv, hq):
    from mini_sglang_mlx_b200 import synthetic as S
    kv_lens = [1, 700, 2500, 33]
    pages = sum((l + 15) // 16 for l in kv_lens)
    w = S.make_decode("heads", hq=hq, hkv=hkv, kv_lens=kv_lens, num_pages=pages + 8, seed=9 + hq, device="cuda")
    assert_close_to_oracle(_run_paged(w), _oracle_for(w), f"decode heads ({hkv}, {hq})")


def test_decode_split_hints_do_not_change_the_result():
    """1, 7, 32 and 128 splits per sequence (the workspace layout's maximum) on the page-granular
    path: the same rows up to fp32 rounding, and the oracle's."""
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, synthetic as S
    kv_lens = [40000, 513, 16, 9000]
    pages = sum((l + 15) // 16 for l in kv_lens)
    w = S.make_decode("hints", hq=16, hkv=4, kv_lens=kv_lens, num_pages=pages + 8, seed=21, device="cuda")
    pip, pidx, lens = w.page_csr()
    ref = _oracle_for(w)
    outs = []
    for hint, mx in ((1, 32), (7, 8), (32, 32), (128, 128)):
        splits = torch.full((len(kv_lens),), hint, dtype=torch.int32, device="cuda")
        out = paged_decode_attention_p16(w.q, w.k_cache, w.v_cache, pip, pidx, lens, splits, w.sm_scale, mx)
        torch.cuda.synchronize()
        assert_close_to_oracle(out, ref, f"decode with {hint} splits")
        outs.append(out.float())
    for o in outs[1:]:
        assert (o - outs[0]).abs().max().item() <= 1.6e-2
