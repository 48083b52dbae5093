"""Seeded random shapes through both index forms of the attention operators against the
oracle: batch, ragged query and prefix lengths (empty sequences included), head counts, the
four mask modes, window sizes, page sizes, element types."""
import math

import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu

HEADS = [(1, 1), (1, 4), (2, 8), (2, 16), (4, 24), (8, 32), (2, 32), (3, 15), (8, 8)]


def _pool(rng, kv_lens, page_size, hkv, d, dtype):
    """A pool of whole pages in random order and the three addressings of the same sequences."""
    need = [(l + page_size - 1) // page_size for l in kv_lens]
    total_pages = sum(need) + 3
    perm = rng.permutation(total_pages)[: sum(need)].astype(np.int32)
    g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    kc = torch.randn(total_pages * page_size, hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(total_pages * page_size, hkv, d, generator=g).to(dtype).cuda()
    slots, off = [], 0
    for l, n in zip(kv_lens, need):
        pages = perm[off:off + n]
        off += n
        t = np.arange(l)
        slots.append(pages[t // page_size].astype(np.int64) * page_size + t % page_size)
    slots = np.concatenate(slots) if slots else np.zeros(0, np.int64)
    pip = torch.from_numpy(O.build_indptr(need)).cuda()
    return (kc, vc, pip, torch.from_numpy(perm).cuda(), torch.from_numpy(slots.astype(np.int32)).cuda(),
            torch.from_numpy(O.build_indptr(kv_lens)).cuda(), torch.tensor(kv_lens, dtype=torch.int32).cuda())


@pytest.mark.parametrize("seed", range(24))
def test_prefill_random_shapes(seed):
    from mini_sglang_mlx_b200 import paged_prefill_attention, paged_prefill_attention_p16
    rng = np.random.default_rng(1000 + seed)
    hkv, hq = HEADS[rng.integers(len(HEADS))]
    d = 256 if seed % 6 == 5 else 128
    dtype = torch.float16 if seed % 5 == 4 else torch.bfloat16
    batch = int(rng.integers(1, 10))
    long_q = seed % 3 == 0
    q_lens = [int(x) for x in rng.integers(0, 400 if long_q else 20, size=batch)]
    if sum(q_lens) == 0:
        q_lens[0] = 7
    prefixes = [int(x) for x in rng.integers(0, 3000, size=batch)]
    cross = bool(rng.integers(2))
    window = int(rng.choice([0, 0, 1, 37, 128, 1000]))
    page_size = int(rng.choice([16, 32]))
    kv_lens = [p + t for p, t in zip(prefixes, q_lens)]
    kc, vc, pip, pidx, slots, kvp, lens = _pool(rng, kv_lens, page_size, hkv, d, dtype)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(sum(q_lens), hq, d, generator=g).to(dtype).cuda()
    qo = torch.from_numpy(O.build_indptr(q_lens)).cuda()
    pre = torch.tensor(prefixes, dtype=torch.int32).cuda()
    scale = 1 / math.sqrt(d)
    kw = dict(is_cross_attention=cross, sliding_window_size=window)
    ref = O.paged_prefill_attention_oracle(q, kc, vc, qo, kvp, slots, pre, scale, **kw)
    what = f"seed {seed}: heads ({hkv},{hq}) d {d} q {q_lens} prefix {prefixes} cross {cross} window {window}"
    out = paged_prefill_attention_p16(q, kc, vc, qo, pip, pidx, lens, pre, scale, max(q_lens),
                                      page_size=page_size, **kw)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, ref, "page-granular, " + what)
    out = paged_prefill_attention(q, kc, vc, qo, kvp, slots, pre, scale, max(q_lens), **kw)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, ref, "per-token, " + what)


@pytest.mark.parametrize("seed", range(12))
def test_decode_random_shapes(seed):
    from mini_sglang_mlx_b200 import paged_decode_attention, paged_decode_attention_p16
    rng = np.random.default_rng(2000 + seed)
    hkv, hq = HEADS[rng.integers(len(HEADS))]
    d = 256 if seed % 4 == 3 else 128
    dtype = torch.float16 if seed % 5 == 4 else torch.bfloat16
    batch = int(rng.integers(1, 20))
    kv_lens = [int(x) for x in rng.integers(0, 6000, size=batch)]
    page_size = int(rng.choice([16, 64]))
    kc, vc, pip, pidx, slots, kvp, lens = _pool(rng, kv_lens, page_size, hkv, d, dtype)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, hq, d, generator=g).to(dtype).cuda()
    splits = torch.from_numpy(rng.integers(1, 33, size=batch).astype(np.int32)).cuda()
    scale = 1 / math.sqrt(d)
    ref = O.paged_decode_attention_oracle(q, kc, vc, kvp, slots, scale)
    what = f"seed {seed}: heads ({hkv},{hq}) d {d} kv {kv_lens}"
    out = paged_decode_attention_p16(q, kc, vc, pip, pidx, lens, splits, scale, 32, page_size=page_size)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, ref, "page-granular, " + what)
    out = paged_decode_attention(q, kc, vc, kvp, slots, splits, scale, 32)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, ref, "per-token, " + what)
