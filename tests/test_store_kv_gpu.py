"""store_kv_cache, the page pool and the backend's metadata on the GPU: exact
(bit-for-bit) against the oracle's scatter and index builders."""
import math

import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("length,hkv,d", [(1, 1, 128), (37, 8, 128), (1000, 4, 128), (64, 2, 256), (5, 3, 100)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scatter_matches_naive_loop(length, hkv, d, dtype):
    from mini_sglang_mlx_b200 import store_kv_cache
    g = torch.Generator().manual_seed(length)
    S = length * 3 + 5
    kc0 = torch.randn(S, hkv, d, generator=g).to(dtype)
    vc0 = torch.randn(S, hkv, d, generator=g).to(dtype)
    k = torch.randn(length, hkv, d, generator=g).to(dtype)
    v = torch.randn(length, hkv, d, generator=g).to(dtype)
    idx = torch.randperm(S, generator=g)[:length].int()
    kc, vc = kc0.clone().cuda(), vc0.clone().cuda()
    store_kv_cache(kc, vc, idx.cuda(), k.cuda(), v.cuda())
    O.store_kv_cache_oracle(kc0, vc0, idx, k, v)
    assert torch.equal(kc.cpu(), kc0) and torch.equal(vc.cpu(), vc0)


def test_scatter_from_a_strided_projection_output():
    # k and v are often two slices of one fused projection: rows are strided
    from mini_sglang_mlx_b200 import store_kv_cache
    hkv, d, n = 4, 128, 50
    kv = torch.randn(n, 2, hkv, d).bfloat16().cuda()
    k, v = kv[:, 0], kv[:, 1]
    kc = torch.zeros(200, hkv, d, dtype=torch.bfloat16).cuda()
    vc = torch.zeros_like(kc)
    idx = torch.randperm(200)[:n].int().cuda()
    store_kv_cache(kc, vc, idx, k, v)
    assert torch.equal(kc[idx.long()], k) and torch.equal(vc[idx.long()], v)


def test_store_rejects_mismatched_inputs():
    from mini_sglang_mlx_b200 import store_kv_cache
    kc = torch.zeros(8, 2, 128, dtype=torch.bfloat16).cuda()
    k = torch.zeros(3, 2, 128, dtype=torch.bfloat16).cuda()
    idx = torch.zeros(3, dtype=torch.int32).cuda()
    with pytest.raises(RuntimeError, match="indices must be int32"):
        store_kv_cache(kc, kc.clone(), idx.long(), k, k)
    with pytest.raises(RuntimeError, match="same dtype"):
        store_kv_cache(kc, kc.clone(), idx, k.half(), k)
    with pytest.raises(RuntimeError, match="shape must be"):
        store_kv_cache(kc, kc.clone(), idx, k[:2], k)


class _Cfg:
    head_dim = 128
    num_kv_heads = 2
    num_qo_heads = 8


def _backend(num_pages=16384, rows=8, max_seq=2048, layers=2):
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    pool = MHAKVCache(_Cfg.num_kv_heads, layers, _Cfg.head_dim, num_pages + 1, torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    # one permutation cut into rows: no slot belongs to two requests (a slot written twice in
    # one scatter has no defined winner on a GPU)
    table = torch.randperm(num_pages, generator=g)[: rows * max_seq].view(rows, max_seq).int().cuda()
    return AttnBackend(_Cfg, pool, table), pool, table


def test_metadata_is_bit_exact_with_the_reference_builders():
    from mini_sglang_mlx_b200.core import Req
    be, _, table = _backend()
    reqs = [Req(table_idx=3, cached_len=100, device_len=164), Req(table_idx=0, cached_len=0, device_len=7),
            Req(table_idx=5, cached_len=999, device_len=1000)]
    md = be.build_prefill_metadata(reqs)
    pos, qo, kvp, idx, pre, mle = O.build_prefill_metadata_oracle(
        table.cpu().numpy(), [r.table_idx for r in reqs], [r.extend_len for r in reqs],
        [r.device_len for r in reqs])
    assert np.array_equal(md.positions.cpu().numpy(), pos)
    assert np.array_equal(md.qo_indptr.cpu().numpy(), qo)
    assert np.array_equal(md.kv_indptr.cpu().numpy(), kvp)
    assert np.array_equal(md.kv_indices.cpu().numpy(), idx)
    assert np.array_equal(md.prefix_lens.cpu().numpy(), pre)
    assert md.max_len_extend == mle
    # virtual K+1-token verify window over the same requests
    md2 = be.build_prefill_metadata(reqs, extend_lens=[8] * 3, kv_lens=[r.cached_len + 8 for r in reqs])
    _, qo2, kvp2, idx2, pre2, _ = O.build_prefill_metadata_oracle(
        table.cpu().numpy(), [r.table_idx for r in reqs], [8] * 3, [r.cached_len + 8 for r in reqs])
    assert np.array_equal(md2.kv_indices.cpu().numpy(), idx2)
    assert np.array_equal(md2.prefix_lens.cpu().numpy(), pre2)
    be.split_policy = "reference"
    dm = be.build_decode_metadata(reqs)
    pos, kvp, idx, splits, mx = O.build_decode_metadata_oracle(
        table.cpu().numpy(), [r.table_idx for r in reqs], [r.device_len for r in reqs],
        [r.cached_len for r in reqs])
    assert np.array_equal(dm.positions.cpu().numpy(), pos)
    assert np.array_equal(dm.kv_indptr.cpu().numpy(), kvp)
    assert np.array_equal(dm.kv_indices.cpu().numpy(), idx)
    assert np.array_equal(dm.num_kv_splits.cpu().numpy(), splits)
    assert dm.max_kv_splits == mx


def test_backend_prefill_then_decode_steps_match_the_oracle():
    """Chunked prefill of three requests, then two decode steps, through
    AttnBackend.forward (store K/V, then attention) on layer 1 of the pool."""
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    be, pool, table = _backend()
    g = torch.Generator().manual_seed(2)
    hq, hkv, d = _Cfg.num_qo_heads, _Cfg.num_kv_heads, _Cfg.head_dim
    layer = 1
    # a shadow pool on the host, written by the oracle's scatter
    kc = torch.zeros(pool.num_pages, hkv, d, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    reqs = [Req(table_idx=1, cached_len=0, device_len=300), Req(table_idx=4, cached_len=0, device_len=45),
            Req(table_idx=6, cached_len=0, device_len=1)]
    phases = [BatchPhase.PREFILL, BatchPhase.DECODE, BatchPhase.DECODE]
    for phase in phases:
        n = sum(r.extend_len for r in reqs)
        q = torch.randn(n, hq, d, generator=g).bfloat16()
        k = torch.randn(n, hkv, d, generator=g).bfloat16()
        v = torch.randn(n, hkv, d, generator=g).bfloat16()
        out_loc = torch.cat([table[r.table_idx, r.cached_len:r.device_len] for r in reqs])
        batch = Batch(reqs=reqs, phase=phase, out_loc=out_loc)
        be.prepare_metadata(batch)
        out = be.forward(q.cuda(), k.cuda(), v.cuda(), layer, batch)
        O.store_kv_cache_oracle(kc, vc, out_loc.cpu(), k, v)
        md = batch.attn_metadata
        if phase == BatchPhase.PREFILL:
            ref = O.paged_prefill_attention_oracle(q, kc, vc, md.qo_indptr, md.kv_indptr, md.kv_indices,
                                                   md.prefix_lens, be.sm_scale)
        else:
            ref = O.paged_decode_attention_oracle(q, kc, vc, md.kv_indptr, md.kv_indices, be.sm_scale)
        assert_close_to_oracle(out, ref, f"backend {phase}")
        for r in reqs:
            r.complete_one()
    assert torch.equal(pool.k_cache(layer).cpu(), kc) and torch.equal(pool.v_cache(layer).cpu(), vc)
    assert torch.count_nonzero(pool.k_cache(0)) == 0


def test_scatter_into_a_pool_beyond_4_gib_per_tensor():
    """Slot ids whose byte offset does not fit in 32 bits (the reference's 32-bit offset
    arithmetic overflows past 2 M slots of 2 KB): rows land where they should, their
    neighbours and the low alias of each offset stay zero."""
    from mini_sglang_mlx_b200 import store_kv_cache
    hkv, d, S = 8, 128, 2_300_000                       # 4.7 GB per tensor
    kc = torch.zeros(S, hkv, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    g = torch.Generator().manual_seed(9)
    idx = torch.tensor([S - 1, 2_097_152, 2_097_153 + 77, 2_200_000, 5], dtype=torch.int32)
    k = torch.randn(len(idx), hkv, d, generator=g).bfloat16().cuda()
    v = torch.randn(len(idx), hkv, d, generator=g).bfloat16().cuda()
    store_kv_cache(kc, vc, idx.cuda(), k, v)
    torch.cuda.synchronize()
    assert torch.equal(kc[idx.long().cuda()], k) and torch.equal(vc[idx.long().cuda()], v)
    assert int((kc != 0).any(dim=(1, 2)).sum()) == len(idx) and int((vc != 0).any(dim=(1, 2)).sum()) == len(idx)


def test_rows_with_an_index_outside_the_pool_are_dropped_and_reported():
    from mini_sglang_mlx_b200 import store_kv_cache
    from mini_sglang_mlx_b200.kernel import device_status
    hkv, d, S = 2, 128, 40
    kc = torch.zeros(S, hkv, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    k = torch.randn(4, hkv, d).bfloat16().cuda()
    v = torch.randn(4, hkv, d).bfloat16().cuda()
    device_status()
    store_kv_cache(kc, vc, torch.tensor([3, S, 7, -1], dtype=torch.int32).cuda(), k, v)
    assert device_status() == 2
    assert torch.equal(kc[3], k[0]) and torch.equal(vc[7], v[2])
    assert int((kc != 0).any(dim=(1, 2)).sum()) == 2          # nothing else was written
    store_kv_cache(kc, vc, torch.tensor([0, 1, 2, 5], dtype=torch.int32).cuda(), k, v)
    assert device_status() == 0


def test_gather_kv_indices_checks_rows_lengths_and_the_output_size():
    from mini_sglang_mlx_b200 import gather_kv_indices
    from mini_sglang_mlx_b200.kernel import device_status
    table = torch.arange(4 * 50, dtype=torch.int32).view(4, 50).cuda()
    indptr = torch.tensor([0, 10, 30], dtype=torch.int32).cuda()
    device_status()
    ok = gather_kv_indices(table, torch.tensor([2, 0], dtype=torch.int32).cuda(), indptr, 30)
    assert device_status() == 0
    assert ok.tolist() == list(range(100, 110)) + list(range(0, 20))
    # a table row that does not exist: skipped and reported, nothing is read
    gather_kv_indices(table, torch.tensor([2, 9], dtype=torch.int32).cuda(), indptr, 30)
    assert device_status() == 2
    # a length beyond the table's columns: clamped and reported
    long = torch.tensor([0, 10, 80], dtype=torch.int32).cuda()
    out = gather_kv_indices(table, torch.tensor([2, 0], dtype=torch.int32).cuda(), long, 80)
    assert device_status() == 2
    assert out[10:60].tolist() == list(range(0, 50))


def test_ops_on_a_stream_that_is_not_the_current_one():
    """``stream=`` runs the kernels (and the first zero-fill of their scratch) on the given
    stream; the caller orders it against the streams that made the inputs."""
    import math
    from mini_sglang_mlx_b200 import paged_decode_attention, paged_prefill_attention
    from oracle import paged_attention_oracle as O
    from tests.helpers import assert_close_to_oracle
    g = torch.Generator().manual_seed(9)
    hkv, hq, d = 2, 8, 128
    kv_lens = [3000, 700]
    total = sum(kv_lens)
    kc = torch.randn(total, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(total, hkv, d, generator=g).bfloat16().cuda()
    slots = torch.randperm(total, generator=g).int().cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    q = torch.randn(2, hq, d, generator=g).bfloat16().cuda()
    splits = torch.tensor([8, 3], dtype=torch.int32).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    out = paged_decode_attention(q, kc, vc, indptr, slots, splits, 1 / math.sqrt(d), 32, stream=side)
    qo = torch.tensor([0, 8, 16], dtype=torch.int32).cuda()
    side.wait_stream(torch.cuda.current_stream())
    qp = torch.randn(16, hq, d, generator=g).bfloat16().cuda()
    pre = torch.tensor([2992, 692], dtype=torch.int32).cuda()
    side.wait_stream(torch.cuda.current_stream())
    outp = paged_prefill_attention(qp, kc, vc, qo, indptr, slots, pre, 1 / math.sqrt(d), 8,
                                   stream=side.cuda_stream)
    side.synchronize()
    assert_close_to_oracle(out, O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, 1 / math.sqrt(d)),
                           "decode on a side stream")
    assert_close_to_oracle(outp, O.paged_prefill_attention_oracle(qp, kc, vc, qo, indptr, slots, pre,
                                                                  1 / math.sqrt(d)),
                           "prefill (key range split) on a side stream")


def test_page_granular_metadata_and_attention_through_the_backend():
    """A backend over page-structured slots (pages of 16 tokens): the metadata carries one id per
    page, attention runs through the page-granular operators, and prefill + decode steps match the
    oracle over the per-token view of the same table."""
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    from mini_sglang_mlx_b200.kernel import device_status
    ps, num_pages, rows, max_seq = 16, 512, 4, 1024
    pool = MHAKVCache(_Cfg.num_kv_heads, 1, _Cfg.head_dim, num_pages * ps, torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    pages = torch.randperm(num_pages, generator=g)[: rows * (max_seq // ps)].view(rows, max_seq // ps)
    table = (pages[:, :, None] * ps + torch.arange(ps)[None, None]).reshape(rows, max_seq).int().cuda()
    be = AttnBackend(_Cfg, pool, table, page_size=ps)
    reqs = [Req(table_idx=2, cached_len=0, device_len=100), Req(table_idx=0, cached_len=0, device_len=33),
            Req(table_idx=3, cached_len=0, device_len=512)]
    device_status()
    md = be.build_prefill_metadata(reqs)
    need = [(r.device_len + ps - 1) // ps for r in reqs]
    assert md.kv_indices is None and md.page_size == ps
    assert md.page_indptr.tolist() == [0, need[0], need[0] + need[1], sum(need)]
    assert md.kv_lens.tolist() == [r.device_len for r in reqs]
    want = torch.cat([pages[r.table_idx, :n] for r, n in zip(reqs, need)])
    assert md.page_indices.cpu().tolist() == want.tolist()
    assert md.qo_indptr.tolist() == [0, 100, 133, 645] and md.prefix_lens.tolist() == [0, 0, 0]
    assert md.positions.cpu().tolist() == sum((list(range(r.device_len)) for r in reqs), [])
    assert device_status() == 0

    scale = 1 / math.sqrt(_Cfg.head_dim)
    n = sum(r.extend_len for r in reqs)
    q = torch.randn(n, _Cfg.num_qo_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
    k = torch.randn(n, _Cfg.num_kv_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
    v = torch.randn(n, _Cfg.num_kv_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
    out_loc = torch.cat([table[r.table_idx, r.cached_len:r.device_len] for r in reqs])
    batch = Batch(reqs=reqs, phase=BatchPhase.PREFILL, out_loc=out_loc)
    be.prepare_metadata(batch)
    out = be.forward(q, k, v, 0, batch)
    kv_lens = [r.device_len for r in reqs]
    slots = torch.cat([table[r.table_idx, : r.device_len] for r in reqs])
    ref = O.paged_prefill_attention_oracle(q, pool.k_cache(0), pool.v_cache(0), md.qo_indptr,
                                           torch.from_numpy(O.build_indptr(kv_lens)), slots,
                                           md.prefix_lens, scale)
    assert_close_to_oracle(out, ref, "prefill through the page-granular backend")
    for _ in range(2):                         # decode steps: one token more per request
        for r in reqs:
            r.complete_one()
        qd = torch.randn(len(reqs), _Cfg.num_qo_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
        kd = torch.randn(len(reqs), _Cfg.num_kv_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
        vd = torch.randn(len(reqs), _Cfg.num_kv_heads, _Cfg.head_dim, generator=g).bfloat16().cuda()
        out_loc = torch.stack([table[r.table_idx, r.cached_len] for r in reqs])
        batch = Batch(reqs=reqs, phase=BatchPhase.DECODE, out_loc=out_loc)
        be.prepare_metadata(batch)
        assert batch.attn_metadata.positions.tolist() == [r.cached_len for r in reqs]
        outd = be.forward(qd, kd, vd, 0, batch)
        kv_lens = [r.device_len for r in reqs]
        slots = torch.cat([table[r.table_idx, : r.device_len] for r in reqs])
        refd = O.paged_decode_attention_oracle(qd, pool.k_cache(0), pool.v_cache(0),
                                               torch.from_numpy(O.build_indptr(kv_lens)), slots, scale)
        assert_close_to_oracle(outd, refd, "decode through the page-granular backend")
    assert device_status() == 0


def test_metadata_kernel_reports_rows_and_lengths_outside_the_table():
    from mini_sglang_mlx_b200.kernel import build_attn_metadata, device_status
    table = torch.arange(4 * 64, dtype=torch.int32).view(4, 64).cuda()
    device_status()
    ok = build_attn_metadata(torch.tensor([[3, 1], [10, 40], [1, 3]], dtype=torch.int32), table,
                             total_q=4, total_kv=50)
    assert device_status() == 0
    assert ok["kv_indptr"].tolist() == [0, 10, 50] and ok["qo_indptr"].tolist() == [0, 3, 4]
    assert ok["kv_indices"].tolist() == list(range(64, 74)) + list(range(192, 232))
    assert ok["positions"].tolist() == [7, 8, 9, 39] and ok["prefix_lens"].tolist() == [7, 39]
    assert ok["num_kv_splits"].tolist() == [1, 1]
    for bad in ([[3, 1], [10, 40], [1, 9]],          # a table row that does not exist
                [[3, 1], [10, 80], [1, 3]],          # longer than a table row
                [[30, 1], [10, 40], [1, 3]]):        # more new tokens than tokens
        build_attn_metadata(torch.tensor(bad, dtype=torch.int32), table, total_q=64, total_kv=128)
        assert device_status() == 2


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_survives():
    """The waits of the attention kernels give up after a limit, raise the CTA's abort flag, set
    the status word to 1 and let the kernel return.  The self-test entry point runs that pattern
    on a barrier nothing completes (limit 200 us here); afterwards the status reads 1 with the
    message of the condition, clears, and the same stream runs an operator correctly."""
    import ctypes
    from mini_sglang_mlx_b200 import _lib, store_kv_cache
    lib = _lib.lib()
    dev = torch.device("cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.msgl_selftest_bounded_wait(ws.data_ptr(), 200, stream) == 0
    word = ctypes.c_int(-1)
    assert lib.msgl_read_status(ws.data_ptr(), 1, ctypes.byref(word), stream) == 7
    assert word.value == 1 and "bounded wait" in _lib.last_error()
    assert lib.msgl_read_status(ws.data_ptr(), 0, ctypes.byref(word), stream) == 0 and word.value == 0
    assert lib.msgl_selftest_bounded_wait(None, 200, stream) == 5
    # the context is intact
    kc = torch.zeros(8, 2, 128, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    k = torch.randn(3, 2, 128, device=dev).bfloat16()
    idx = torch.tensor([5, 0, 2], dtype=torch.int32, device=dev)
    store_kv_cache(kc, vc, idx, k, k)
    torch.cuda.synchronize()
    assert torch.equal(kc[idx.long()], k)
