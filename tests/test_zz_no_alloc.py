"""The allocation-free decode entry point against the ordinary one.

``msgl_paged_decode_attention_static`` serves callers that cannot hand the
library a workspace because they cannot allocate device memory where they
call it (a fixed memory budget, a device heap owned by another runtime).  It
must give the result of ``msgl_paged_decode_attention`` on the same inputs;
the test calls it twice in a row through the C ABI, with a different problem
in between, because both calls share one built-in scratch array that keeps
the previous call's contents.  The file name sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import math

import pytest
import torch

from mini_sglang_mlx_b200 import _lib
from oracle import paged_attention_oracle as O
from tests.helpers import MAX_ABS_TOL, MEAN_ABS_TOL, assert_close_to_oracle


def _problem(kv_lens, hkv, hq, seed, d=128):
    g = torch.Generator().manual_seed(seed)
    total = sum(kv_lens)
    kc = torch.randn(total + 3, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(total + 3, hkv, d, generator=g).bfloat16().cuda()
    q = torch.randn(len(kv_lens), hq, d, generator=g).bfloat16().cuda()
    slots = torch.randperm(total + 3, generator=g)[:total].int().cuda()
    indptr = torch.from_numpy(O.build_indptr(kv_lens)).cuda()
    splits = torch.from_numpy(O.compute_num_kv_splits(kv_lens)).cuda()
    return q, kc, vc, indptr, slots, splits


def _static(q, kc, vc, indptr, slots, splits, max_splits=32):
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    rc = _lib.lib().msgl_paged_decode_attention_static(
        q.data_ptr(), kc.data_ptr(), vc.data_ptr(), indptr.data_ptr(), slots.data_ptr(),
        splits.data_ptr(), out.data_ptr(), q.shape[0], q.shape[1], kc.shape[1], q.shape[2],
        kc.shape[0], _lib.DTYPE_BF16, 1 / math.sqrt(q.shape[2]), max_splits, stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out


@pytest.mark.gpu
def test_static_scratch_entry_matches_the_workspace_entry_twice_in_a_row():
    from mini_sglang_mlx_b200 import paged_decode_attention
    first = _problem([3000, 1, 517, 129], 8, 16, seed=1)
    second = _problem([64, 4100], 2, 8, seed=2)          # different shape: stale partials in the array
    for args in (first, second, first):
        ref = paged_decode_attention(*args, 1 / math.sqrt(128), 32)
        got = _static(*args)
        diff = (got.float() - ref.float()).abs()
        assert diff.max() <= MAX_ABS_TOL and diff.mean() <= MEAN_ABS_TOL
        assert_close_to_oracle(got, O.paged_decode_attention_oracle(*args[:5], 1 / math.sqrt(128)),
                               "static-scratch decode")


@pytest.mark.gpu
def test_static_scratch_entry_reports_a_slot_outside_the_pool():
    """The status word of the built-in array is read (and cleared) with msgl_read_status(NULL)."""
    import ctypes
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    word = ctypes.c_int(-1)
    assert lib.msgl_read_status(None, 1, ctypes.byref(word), stream) in (0, 7)   # start clean
    q, kc, vc, indptr, slots, splits = _problem([600, 70], 2, 8, seed=3)
    bad = slots.clone()
    bad[5] = kc.shape[0] + 11
    got = _static(q, kc, vc, indptr, bad, splits)
    assert torch.isfinite(got.float()).all()
    assert lib.msgl_read_status(None, 1, ctypes.byref(word), stream) == 7 and word.value == 2
    assert "outside the pool" in _lib.last_error()
    _static(q, kc, vc, indptr, slots, splits)
    assert lib.msgl_read_status(None, 0, ctypes.byref(word), stream) == 0 and word.value == 0


def test_static_scratch_entry_rejects_problems_beyond_its_array():
    # 4096 * 32 * 32 partial rows need far more than the 32 MiB the library holds;
    # the check needs no device, so it also runs where there is no GPU
    rc = _lib.lib().msgl_paged_decode_attention_static(
        None, None, None, None, None, None, None, 4096, 32, 8, 128, 1 << 20, _lib.DTYPE_BF16, 0.1, 32,
        None)
    assert rc == 5
    msg = _lib.last_error()
    assert "paged_decode_attention_static" in msg and str(_lib.STATIC_SCRATCH_BYTES) in msg
