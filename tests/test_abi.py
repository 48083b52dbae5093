"""The C-ABI library loads, exports what the header declares and rejects bad
arguments with the documented status codes — no kernel is launched here."""
import ctypes
import re
from pathlib import Path

import pytest

from mini_sglang_mlx_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "msgl_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msgl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for name in ("msgl_paged_decode_attention", "msgl_paged_prefill_attention", "msgl_store_kv_cache",
                 "msgl_decode_workspace_bytes", "msgl_prefill_workspace_bytes",
                 "msgl_gather_kv_indices", "msgl_last_error_string", "msgl_abi_version"):
        assert name in syms


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    # and the ctypes table covers every declaration
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_abi_version():
    assert _lib.lib().msgl_abi_version() == 2


def test_decode_workspace_bytes():
    lib = _lib.lib()
    # header (status word + arrival counters) + fp32 partials (B,Hq,S,D) + fp32 lse (B,Hq,S)
    header = 256 + 16384 * 4
    assert lib.msgl_decode_workspace_bytes(8, 16, 128, 32) == header + 8 * 16 * 32 * 129 * 4
    assert lib.msgl_decode_workspace_bytes(0, 16, 128, 32) == header
    # more (sequence, head) pairs than the header has counters: a counter region of their own
    big = lib.msgl_decode_workspace_bytes(2048, 16, 128, 2)
    assert big == header + 2048 * 16 * 4 + 2048 * 16 * 2 * 129 * 4


DEC_OK = dict(batch=2, hq=16, hkv=8, d=128, slots=64, dtype=0, splits=32)


def call_decode(**kw):
    a = dict(DEC_OK, **kw)
    return _lib.lib().msgl_paged_decode_attention(
        None, None, None, None, None, None, None, None, 0, a["batch"], a["hq"], a["hkv"], a["d"],
        a["slots"], a["dtype"], 0.1, a["splits"], None)


@pytest.mark.parametrize("kw,code,text", [
    (dict(d=64), 3, "paged_decode_attention: head_dim must be 128 or 256"),
    (dict(hq=12, hkv=8), 4, "paged_decode_attention: num_q_heads must be a multiple of num_kv_heads"),
    (dict(hq=34, hkv=2), 4, "paged_decode_attention: only q_heads/kv_heads <= 16 is supported"),
    (dict(dtype=9), 2, "paged_decode_attention: unsupported dtype, must be float16 or bfloat16"),
    (dict(splits=0), 5, "max_kv_splits"),
    (dict(), 5, "null tensor pointer"),
])
def test_decode_rejects_bad_arguments(kw, code, text):
    assert call_decode(**kw) == code
    assert text in _lib.last_error()


def test_decode_empty_batch_is_a_no_op():
    assert call_decode(batch=0) == 0


def call_prefill(batch=2, total_q=8, hq=32, hkv=8, d=128, dtype=0, window=0):
    return _lib.lib().msgl_paged_prefill_attention(
        None, None, None, None, None, None, None, None, None, 0, batch, total_q, 100, hq, hkv, d, 64,
        dtype, 0.1, 4, 0, window, None)


@pytest.mark.parametrize("kw,code,text", [
    (dict(d=96), 3, "paged_prefill_attention: head_dim must be 128 or 256"),
    (dict(hq=30), 4, "paged_prefill_attention: num_q_heads must be a multiple of num_kv_heads"),
    (dict(window=-1), 5, "paged_prefill_attention: sliding_window_size must be >= 0"),
    (dict(batch=0), 1, "paged_prefill_attention: batch must be > 0"),
    (dict(dtype=5), 2, "paged_prefill_attention: unsupported dtype"),
    (dict(), 5, "null tensor pointer"),
])
def test_prefill_rejects_bad_arguments(kw, code, text):
    assert call_prefill(**kw) == code
    assert text in _lib.last_error()


def test_attention_ops_reject_misaligned_tensors():
    """Pointers are only compared here, never followed: the check comes before any CUDA call."""
    lib = _lib.lib()
    ok, odd = 0x10000, 0x10008
    assert lib.msgl_paged_decode_attention(odd, ok, ok, ok, ok, None, ok, ok, 1 << 20, 2, 16, 8, 128, 64,
                                           0, 0.1, 4, None) == 5
    assert "16-byte aligned" in _lib.last_error()
    assert lib.msgl_paged_prefill_attention(ok, ok, odd, ok, ok, ok, ok, ok, ok, 1 << 20, 2, 8, 100, 32, 8,
                                            128, 64, 0, 0.1, 4, 0, 0, None) == 5
    assert "16-byte aligned" in _lib.last_error()


def test_prefill_launch_count_is_host_arithmetic():
    lib = _lib.lib()
    # a 512-token chunk per sequence fills the GPU with query tiles: one launch
    assert lib.msgl_prefill_launch_count(4, 2048, 16000, 32, 8, 128, 512, 0, 1) == 1
    # 128 query tokens over 32768 keys: split in many pieces of 256 rows, merged by a second launch
    assert lib.msgl_prefill_launch_count(1, 128, 32896, 32, 8, 128, 128, 0, 1) == 2
    # a 16-token draft block over a window: small units, merged inside the launch
    assert lib.msgl_prefill_launch_count(16, 256, 16 * 8192, 32, 8, 128, 16, 4096, 1) == 1


def test_store_rejects_bad_arguments():
    lib = _lib.lib()
    assert lib.msgl_store_kv_cache(None, None, None, None, None, 4, 8, 126, 64, 8 * 126, 8 * 126, 0, None, None) == 1
    assert "store_kv_cache: head_dim must be a multiple of 4" in _lib.last_error()
    assert lib.msgl_store_kv_cache(None, None, None, None, None, 4, 8, 128, 64, 8 * 128, 8 * 128, 7, None, None) == 2
    assert lib.msgl_store_kv_cache(None, None, None, None, None, 0, 8, 128, 64, 8 * 128, 8 * 128, 0, None, None) == 0


def test_python_ops_refuse_cpu_tensors():
    import torch
    from mini_sglang_mlx_b200 import paged_decode_attention
    q = torch.zeros(1, 2, 128, dtype=torch.bfloat16)
    kc = torch.zeros(4, 1, 128, dtype=torch.bfloat16)
    z = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        paged_decode_attention(q, kc, kc, z, z, z[:1], 0.1, 32)
    with pytest.raises(RuntimeError, match="q must be 3D"):
        paged_decode_attention(q[0], kc, kc, z, z, z[:1], 0.1, 32)


def test_prefill_workspace_follows_the_split_policy():
    """No kernel launch: the scratch size tells whether the key range will be split.  Query tiles
    that already fill more than half of the CTA slots run unsplit (status area only); verify and
    draft-block shapes and small chunks over long prefixes get partials for a merge pass."""
    ws = _lib.lib().msgl_prefill_workspace_bytes
    status_only = ws(1, 0, 0, 32, 8, 128, 0, 0)
    # chunked prefill, 4 x 512 query tokens, Hq32/Hkv8: 256 query tiles -> no split
    assert ws(4, 2048, 12000, 32, 8, 128, 512, 0) == status_only
    # speculative verify: 32 sequences x 8 tokens over ~300k keys, Hkv 4: 128 tiles of 296 slots -> split
    verify = ws(32, 256, 303560, 32, 4, 128, 8, 0)
    assert verify > status_only
    # one 128-token chunk over a 32k prefix: 16 tiles -> split into many pieces
    assert ws(1, 128, 32896, 32, 8, 128, 128, 0) > status_only
    # more keys never need less scratch
    assert ws(32, 256, 607120, 32, 4, 128, 8, 0) >= verify
    # head_dim 256 runs one CTA per SM: 128 (sequence, head) units already fill most of 148 slots
    # (no split), 32 units do not
    assert ws(32, 256, 303560, 32, 4, 256, 8, 0) == status_only
    assert ws(8, 64, 75890, 32, 4, 256, 8, 0) > status_only


def test_page_granular_workspace_queries_are_host_arithmetic():
    lib = _lib.lib()
    idx = lib.msgl_page_index_workspace_bytes(4, 1000, 16)
    assert idx == ((4 + 1 + 16000) * 4 + 255) // 256 * 256
    assert lib.msgl_page_index_workspace_bytes(0, 0, 16) == 256
    op = lib.msgl_prefill_workspace_bytes(4, 2048, 16000, 32, 8, 128, 512, 0)
    both = lib.msgl_prefill_workspace_bytes_p16(4, 2048, 1000, 16, 32, 8, 128, 512, 0)
    assert both == (op + 255) // 256 * 256 + idx
