"""The attention ops inside a CUDA graph: captured once, replayed on new input contents.

The ops launch on the current stream without host synchronisation and take their scratch from
a per-stream cache, so a capture records exactly their kernels; a replay must give the result
of an eager call on the same inputs, bit for bit.
"""
import math

import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu


def _capture(fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()                                   # scratch and kernel attributes set up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fn()
    return graph, out


def test_decode_replays_on_new_contents():
    from mini_sglang_mlx_b200 import paged_decode_attention
    g = torch.Generator().manual_seed(1)
    kv_lens = [300, 1, 2048, 777]
    hkv, hq, d = 8, 16, 128
    total = sum(kv_lens)
    kc = torch.randn(total + 3, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(total + 3, hkv, d, generator=g).bfloat16().cuda()
    q = torch.randn(len(kv_lens), hq, d, generator=g).bfloat16().cuda()
    slots = torch.randperm(total + 3, generator=g)[:total].int().cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
    scale = 1 / math.sqrt(d)
    call = lambda: paged_decode_attention(q, kc, vc, indptr, slots, splits, scale, 32)  # noqa: E731
    graph, out = _capture(call)
    for seed in (2, 3):
        gq = torch.Generator().manual_seed(seed)
        q.copy_(torch.randn(q.shape, generator=gq).bfloat16())
        kc.copy_(torch.randn(kc.shape, generator=gq).bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, call())
        assert_close_to_oracle(out, O.paged_decode_attention_oracle(q, kc, vc, indptr, slots, scale),
                               f"decode graph replay {seed}")


@pytest.mark.parametrize("q_lens,prefix", [([64, 200], [100, 0]), ([8, 8], [3000, 5000]), ([128], [20000])],
                         ids=str)
def test_prefill_replays_on_new_contents(q_lens, prefix):
    """Unsplit, split with the merge inside the launch, and split with the merge as a second,
    programmatically dependent launch (both launches are captured)."""
    from mini_sglang_mlx_b200 import _lib, paged_prefill_attention
    g = torch.Generator().manual_seed(5)
    hkv, hq, d = 2, 8, 128
    kv_lens = [p + t for p, t in zip(prefix, q_lens)]
    launches = _lib.lib().msgl_prefill_launch_count(len(q_lens), sum(q_lens), sum(kv_lens), hq, hkv, d,
                                                    max(q_lens), 0, 0)
    assert launches == (2 if q_lens == [128] else 1)
    total = sum(kv_lens)
    kc = torch.randn(total + 9, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(total + 9, hkv, d, generator=g).bfloat16().cuda()
    q = torch.randn(sum(q_lens), hq, d, generator=g).bfloat16().cuda()
    slots = torch.randperm(total + 9, generator=g)[:total].int().cuda()
    qo = torch.from_numpy(O.build_indptr(q_lens)).cuda()
    kvp = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    pre = torch.tensor(prefix, dtype=torch.int32).cuda()
    scale = 1 / math.sqrt(d)
    call = lambda: paged_prefill_attention(q, kc, vc, qo, kvp, slots, pre, scale, max(q_lens))  # noqa: E731
    graph, out = _capture(call)
    gq = torch.Generator().manual_seed(6)
    q.copy_(torch.randn(q.shape, generator=gq).bfloat16())
    vc.copy_(torch.randn(vc.shape, generator=gq).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, call())
    assert_close_to_oracle(out, O.paged_prefill_attention_oracle(q, kc, vc, qo, kvp, slots, pre, scale),
                           f"prefill graph replay {q_lens}")
