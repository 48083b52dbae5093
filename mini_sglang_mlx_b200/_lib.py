"""ctypes binding of ``libmsgl_b200.so`` (declarations: ``include/msgl_b200.h``).

The library is the product: there is no Python or CPU fallback.  If the shared
object is missing, loading raises with the build command.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmsgl_b200.so"

MSGL_OK = 0
DTYPE_BF16 = 0
DTYPE_F16 = 1
MAX_KV_SPLITS_LIMIT = 128
STATIC_SCRATCH_BYTES = 32 << 20

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol of include/msgl_b200.h
SIGNATURES = {
    "msgl_abi_version": (_i, []),
    "msgl_last_error_string": (C.c_char_p, []),
    "msgl_device_sm_count": (_i, []),
    "msgl_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "msgl_paged_decode_attention": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i64, _i, _f, _i, _vp]),
    "msgl_paged_decode_attention_gated": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i64, _i, _f, _i, _vp]),
    "msgl_paged_prefill_attention_gated": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i64, _i, _i, _i, _i64,
             _i, _f, _i, _i, _i, _vp]),
    "msgl_paged_decode_attention_static": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _f, _i, _vp]),
    "msgl_read_status": (_i, [_vp, _i, _vp, _vp]),
    "msgl_prefill_workspace_bytes": (_sz, [_i, _i, _i64, _i, _i, _i, _i, _i]),
    "msgl_selftest_bounded_wait": (_i, [_vp, _i, _vp]),
    "msgl_prefill_launch_count": (_i, [_i, _i, _i64, _i, _i, _i, _i, _i, _i]),
    "msgl_page_index_workspace_bytes": (_sz, [_i, _i64, _i]),
    "msgl_paged_decode_attention_p16": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i64, _i, _f, _i,
             _i, _i64, _vp]),
    "msgl_build_attn_metadata": (
        _i, [_vp, _vp, _i64, _i64, _i64, _i, _i, _i, _i, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp,
             _vp, _vp, _vp, _vp, _vp]),
    "msgl_prefill_workspace_bytes_p16": (_sz, [_i, _i, _i64, _i, _i, _i, _i, _i, _i]),
    "msgl_paged_prefill_attention_p16": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i64, _i,
             _f, _i, _i, _i, _i, _i64, _vp]),
    "msgl_paged_prefill_attention": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i64, _i, _i, _i, _i64,
             _i, _f, _i, _i, _i, _vp]),
    "msgl_store_kv_cache": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "msgl_gather_kv_indices": (_i, [_vp, _i64, _vp, _vp, _vp, _i, _i64, _i64, _i64, _vp, _vp]),
    "msgl_fast_compare_key": (_i64, [_vp, _vp, _i64, _i64, _i]),
    "msgl_qk_norm_rope_store": (
        _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _i64, _i64,
             _i64, _i64, _i64, _i, _vp]),
}


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mini_sglang_mlx_b200.build` "
            "(there is no fallback implementation)")
    handle = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    return handle


def last_error() -> str:
    return lib().msgl_last_error_string().decode()


def check(status: int) -> None:
    """Raise RuntimeError with the library's message (same prefixes as the
    reference wrappers' std::runtime_error texts) on a non-OK status."""
    if status != MSGL_OK:
        raise RuntimeError(f"{last_error()} [msgl status {status}]")
