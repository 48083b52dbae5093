"""Page-granular index entries (one id per page of page_size tokens) on the GPU.

The reference has one token per page (mini_sglang_mlx/engine/engine.py:103) and per-token
``kv_indices``; these entries take (page_indptr, page_indices, kv_lens) instead.  Checked
against the per-token ops on the same pool (decode: bit-exact, same kernels and indices) and
against the fp32 oracle.
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


@pytest.mark.parametrize("page_size", [1, 16, 64])
@pytest.mark.parametrize("kv_lens", [[1], [237, 809], [16, 32, 48], [0, 5, 0, 4097], [2048] * 3 + [1]],
                         ids=str)
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


@pytest.mark.parametrize("page_size", [1, 16])
@pytest.mark.parametrize("case", [
    dict(q_lens=[5, 17], prefix=[0, 40]),
    dict(q_lens=[512], prefix=[1000]),
    dict(q_lens=[16] * 4, prefix=[3000, 100, 0, 2047], window=1024),
    dict(q_lens=[8, 8], prefix=[4000, 6000]),                       # short block: key range is split
    dict(q_lens=[33, 1], prefix=[64, 64], cross=True),
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
        q.data_ptr(), ws.data_ptr(), ws.numel(), 3, 4, 2, 128, 1600, _lib.DTYPE_BF16, 0.1, 32, 16, 100, 0)
    assert rc != 0 and "workspace too small" in lib.msgl_last_error_string().decode()
