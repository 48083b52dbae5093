"""Operators of the reference extension ``mini_sglang_mlx_kernel`` on B200.

Same names, argument order and keyword arguments as the reference bindings
(mini-sglang-mlx-kernel/csrc/bindings.cpp:27-55), with ``mx.array`` replaced by
CUDA ``torch.Tensor``.  Each call validates what only the tensor objects can
tell (rank, dtype, device, contiguity), hands raw pointers to the C-ABI
library on the current (or given) CUDA stream and returns without a host
synchronisation.  Errors surface as ``RuntimeError`` with the reference's
op-prefixed messages.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import _lib

__all__ = [
    "paged_decode_attention",
    "paged_prefill_attention",
    "paged_decode_attention_p16",
    "paged_prefill_attention_p16",
    "store_kv_cache",
    "gather_kv_indices",
    "fast_compare_key",
    "qk_norm_rope_store",
    "build_attn_metadata",
    "device_status",
]

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}

# scratch per (device index, stream handle, operator); grown on demand, never shrunk.  The
# operators keep arrival counters in their scratch that must read zero when a call starts (the
# kernels put them back to zero), so a buffer is zero-filled once, on the stream that will use
# it, and never shared between operators.
_workspaces: Dict[Tuple[int, int, str], torch.Tensor] = {}
_retired: list = []   # outgrown buffers stay alive: work queued on their stream may still use them


_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_handle(stream, device: torch.device) -> int:
    if stream is None:
        # (the raw getter skips the construction of a Stream object: a few microseconds per call)
        if _raw_current_stream is not None:
            return _raw_current_stream(device.index if device.index is not None
                                       else torch.cuda.current_device())
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


class _NoCtx:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_CTX = _NoCtx()


def _on_device(device: torch.device):
    """Context that makes ``device`` current for the launches inside; nothing to do (and nothing
    to pay) when it already is."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_CTX
    return torch.cuda.device(device)


def _workspace(nbytes: int, device: torch.device, stream_handle: int, kind: str) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, stream_handle, kind)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
        # allocated and zero-filled on the stream the kernels will run on, so that the fill is
        # ordered before them even when that stream is not torch's current one
        with torch.cuda.stream(torch.cuda.ExternalStream(stream_handle, device=device)):
            ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def device_status(device=None) -> int:
    """Synchronise and return the OR of the device status words of every
    workspace on ``device`` (0 = no kernel reported an out-of-range slot),
    clearing them."""
    torch.cuda.synchronize(device)
    status = 0
    for ws in _workspaces.values():
        word = ws[:4].view(torch.int32)
        status |= int(word.item())
        word.zero_()
    return status


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_common(op: str, q, k_cache, v_cache, index_arrays, index_msg: str, q_msg: str):
    _require(q.dim() == 3, f"{op}: {q_msg}")
    _require(k_cache.dim() == 3 and v_cache.dim() == 3,
             f"{op}: k_cache and v_cache must be 3D (num_pages, num_kv_heads, head_dim)")
    _require(all(a.dim() == 1 for a in index_arrays), f"{op}: {index_msg}")
    _require(q.is_cuda, f"{op}: tensors must live on a CUDA device")
    for t in (k_cache, v_cache, *index_arrays):
        _require(t.device == q.device, f"{op}: all tensors must be on the same device")
    _require(q.dtype in _DTYPES, f"{op}: unsupported dtype, must be float16 or bfloat16")
    _require(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype,
             f"{op}: q, k_cache and v_cache must have the same dtype")
    for a in index_arrays:
        _require(a.dtype == torch.int32, f"{op}: index arrays must be int32")
        _require(a.is_contiguous(), f"{op}: index arrays must be contiguous")
    _require(q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(),
             f"{op}: q, k_cache and v_cache must be contiguous")
    _require(k_cache.shape == v_cache.shape, f"{op}: v_cache shape must match k_cache")


def _check_gate(op: str, gate, q) -> None:
    _require(gate.shape == q.shape and gate.dtype == q.dtype and gate.device == q.device
             and gate.is_contiguous(), f"{op}: gate must match q in shape, dtype and device, contiguous")


def paged_decode_attention(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits,
                           sm_scale: float, max_kv_splits: int, *, gate=None,
                           stream=None) -> torch.Tensor:
    """Decode attention of one query token per sequence over its paged KV.

    q ``(batch, Hq, D)``; caches ``(num_slots, Hkv, D)``; ``kv_indptr``
    ``(batch+1)``, ``kv_indices`` ``(total_kv)``, ``num_kv_splits`` ``(batch)``
    int32.  Returns ``(batch, Hq, D)`` in q's dtype.  Signature of the
    reference op: mini-sglang-mlx-kernel/csrc/bindings.cpp:36-44.  ``gate`` (not in the
    reference op; same shape as q) fuses the ``* sigmoid(gate)`` of the reference's Qwen3.5
    attention layer (models/qwen3_5.py:110) into the final write.
    """
    op = "paged_decode_attention"
    _check_common(op, q, k_cache, v_cache, (kv_indptr, kv_indices, num_kv_splits),
                  "kv_indptr, kv_indices, num_kv_splits must be 1D",
                  "q must be 3D (batch, num_q_heads, head_dim)")
    batch, hq, d = q.shape
    _require(k_cache.shape[2] == d, f"{op}: cache head_dim must match q head_dim")
    _require(kv_indptr.numel() == batch + 1 and num_kv_splits.numel() == batch,
             f"{op}: kv_indptr must have batch+1 and num_kv_splits batch entries")
    out = torch.empty_like(q)
    sh = _stream_handle(stream, q.device)
    lib = _lib.lib()
    with _on_device(q.device):
        need = lib.msgl_decode_workspace_bytes(batch, hq, d, int(max_kv_splits))
        ws = _workspace(need, q.device, sh, "decode")
        tail = (out.data_ptr(), ws.data_ptr(), ws.numel(), batch, hq, k_cache.shape[1], d,
                k_cache.shape[0], _DTYPES[q.dtype], float(sm_scale), int(max_kv_splits), sh)
        head = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), kv_indptr.data_ptr(),
                kv_indices.data_ptr(), num_kv_splits.data_ptr())
        if gate is None:
            _lib.check(lib.msgl_paged_decode_attention(*head, *tail))
        else:
            _check_gate(op, gate, q)
            _lib.check(lib.msgl_paged_decode_attention_gated(*head, gate.data_ptr(), *tail))
    return out


def paged_prefill_attention(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, prefix_lens,
                            sm_scale: float, max_len_extend: int, *,
                            is_cross_attention: bool = False, sliding_window_size: int = 0,
                            gate=None, stream=None) -> torch.Tensor:
    """Ragged multi-token attention over prefix + extend tokens of paged KV.

    q ``(total_q, Hq, D)``; ``qo_indptr``/``kv_indptr`` ``(batch+1)``,
    ``kv_indices`` ``(total_kv)``, ``prefix_lens`` ``(batch)`` int32.  Mask:
    causal by default; ``is_cross_attention`` drops the causal bound;
    ``sliding_window_size`` W > 0 keeps keys at positions >= pos - W + 1.
    Signature of the reference op: mini-sglang-mlx-kernel/csrc/bindings.cpp:45-55.
    ``gate`` (not in the reference op; same shape as q): out = attention * sigmoid(gate).
    """
    op = "paged_prefill_attention"
    _check_common(op, q, k_cache, v_cache, (qo_indptr, kv_indptr, kv_indices, prefix_lens),
                  "qo_indptr, kv_indptr, kv_indices, prefix_lens must be 1D",
                  "q must be 3D (total_q_tokens, num_q_heads, head_dim)")
    total_q, hq, d = q.shape
    _require(k_cache.shape[2] == d, f"{op}: cache head_dim must match q head_dim")
    batch = qo_indptr.numel() - 1
    _require(batch > 0, f"{op}: batch must be > 0")
    _require(kv_indptr.numel() == batch + 1 and prefix_lens.numel() == batch,
             f"{op}: kv_indptr must have batch+1 and prefix_lens batch entries")
    out = torch.empty_like(q)
    sh = _stream_handle(stream, q.device)
    lib = _lib.lib()
    total_kv = kv_indices.numel()
    with _on_device(q.device):
        need = lib.msgl_prefill_workspace_bytes(batch, total_q, total_kv, hq, k_cache.shape[1], d,
                                                int(max_len_extend), int(sliding_window_size))
        ws = _workspace(need, q.device, sh, "prefill")
        head = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), qo_indptr.data_ptr(),
                kv_indptr.data_ptr(), kv_indices.data_ptr(), prefix_lens.data_ptr())
        tail = (out.data_ptr(), ws.data_ptr(), ws.numel(), batch, total_q, total_kv, hq, k_cache.shape[1],
                d, k_cache.shape[0], _DTYPES[q.dtype], float(sm_scale), int(max_len_extend),
                int(bool(is_cross_attention)), int(sliding_window_size), sh)
        if gate is None:
            _lib.check(lib.msgl_paged_prefill_attention(*head, *tail))
        else:
            _check_gate(op, gate, q)
            _lib.check(lib.msgl_paged_prefill_attention_gated(*head, gate.data_ptr(), *tail))
    return out


def paged_decode_attention_p16(q, k_cache, v_cache, page_indptr, page_indices, kv_lens, num_kv_splits,
                               sm_scale: float, max_kv_splits: int, *, page_size: int = 16,
                               gate=None, stream=None) -> torch.Tensor:
    """``paged_decode_attention`` for a pool allocated in pages of ``page_size`` tokens
    (slot = page * page_size + offset): ``page_indptr`` ``(batch+1)``, ``page_indices``
    ``(total_pages)`` and the token lengths ``kv_lens`` ``(batch)`` replace the per-token
    ``kv_indptr`` / ``kv_indices`` of the reference op (the reference hard-wires one token per
    page, mini_sglang_mlx/engine/engine.py:103).  No host synchronisation: the per-token ids
    are built on the device in front of the same kernels."""
    op = "paged_decode_attention_p16"
    _check_common(op, q, k_cache, v_cache, (page_indptr, page_indices, kv_lens, num_kv_splits),
                  "page_indptr, page_indices, kv_lens, num_kv_splits must be 1D",
                  "q must be 3D (batch, num_q_heads, head_dim)")
    batch, hq, d = q.shape
    _require(k_cache.shape[2] == d, f"{op}: cache head_dim must match q head_dim")
    _require(page_indptr.numel() == batch + 1 and kv_lens.numel() == batch
             and num_kv_splits.numel() == batch,
             f"{op}: page_indptr must have batch+1, kv_lens and num_kv_splits batch entries")
    _require(int(page_size) > 0, f"{op}: page_size must be > 0")
    out = torch.empty_like(q)
    sh = _stream_handle(stream, q.device)
    lib = _lib.lib()
    total_pages = page_indices.numel()
    with _on_device(q.device):
        need = ((lib.msgl_decode_workspace_bytes(batch, hq, d, int(max_kv_splits)) + 255) // 256 * 256
                + lib.msgl_page_index_workspace_bytes(batch, total_pages, int(page_size)))
        ws = _workspace(need, q.device, sh, "decode")
        if gate is not None:
            _check_gate(op, gate, q)
        _lib.check(lib.msgl_paged_decode_attention_p16(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_indptr.data_ptr(),
            page_indices.data_ptr(), kv_lens.data_ptr(), num_kv_splits.data_ptr(),
            gate.data_ptr() if gate is not None else None, out.data_ptr(),
            ws.data_ptr(), ws.numel(), batch, hq, k_cache.shape[1], d, k_cache.shape[0],
            _DTYPES[q.dtype], float(sm_scale), int(max_kv_splits), int(page_size), total_pages, sh))
    return out


def paged_prefill_attention_p16(q, k_cache, v_cache, qo_indptr, page_indptr, page_indices, kv_lens,
                                prefix_lens, sm_scale: float, max_len_extend: int, *,
                                page_size: int = 16, is_cross_attention: bool = False,
                                sliding_window_size: int = 0, gate=None, stream=None) -> torch.Tensor:
    """``paged_prefill_attention`` with one id per page of ``page_size`` tokens instead of one
    per token; see ``paged_decode_attention_p16``."""
    op = "paged_prefill_attention_p16"
    _check_common(op, q, k_cache, v_cache, (qo_indptr, page_indptr, page_indices, kv_lens, prefix_lens),
                  "qo_indptr, page_indptr, page_indices, kv_lens, prefix_lens must be 1D",
                  "q must be 3D (total_q_tokens, num_q_heads, head_dim)")
    total_q, hq, d = q.shape
    _require(k_cache.shape[2] == d, f"{op}: cache head_dim must match q head_dim")
    batch = qo_indptr.numel() - 1
    _require(batch > 0, f"{op}: batch must be > 0")
    _require(page_indptr.numel() == batch + 1 and kv_lens.numel() == batch
             and prefix_lens.numel() == batch,
             f"{op}: page_indptr must have batch+1, kv_lens and prefix_lens batch entries")
    _require(int(page_size) > 0, f"{op}: page_size must be > 0")
    out = torch.empty_like(q)
    sh = _stream_handle(stream, q.device)
    lib = _lib.lib()
    total_pages = page_indices.numel()
    with _on_device(q.device):
        need = lib.msgl_prefill_workspace_bytes_p16(batch, total_q, total_pages, int(page_size), hq,
                                                    k_cache.shape[1], d, int(max_len_extend),
                                                    int(sliding_window_size))
        ws = _workspace(need, q.device, sh, "prefill")
        if gate is not None:
            _check_gate(op, gate, q)
        _lib.check(lib.msgl_paged_prefill_attention_p16(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), qo_indptr.data_ptr(),
            page_indptr.data_ptr(), page_indices.data_ptr(), kv_lens.data_ptr(), prefix_lens.data_ptr(),
            gate.data_ptr() if gate is not None else None,
            out.data_ptr(), ws.data_ptr(), ws.numel(), batch, total_q, hq, k_cache.shape[1], d,
            k_cache.shape[0], _DTYPES[q.dtype], float(sm_scale), int(max_len_extend),
            int(bool(is_cross_attention)), int(sliding_window_size), int(page_size), total_pages, sh))
    return out


def store_kv_cache(k_cache, v_cache, indices, k, v, *, stream=None) -> None:
    """In place: ``k_cache[indices[r]] = k[r]``, ``v_cache[indices[r]] = v[r]``.

    Signature and checks of the reference op:
    mini-sglang-mlx-kernel/csrc/bindings.cpp:27-32, csrc/store_kv_cache.cpp:22-63.
    """
    op = "store_kv_cache"
    _require(k_cache.dim() == 3 and v_cache.dim() == 3,
             f"{op}: k_cache and v_cache must be 3D (num_pages, num_kv_heads, head_dim)")
    _require(indices.dim() == 1, f"{op}: indices must be 1D")
    _require(k.dim() == 3 and v.dim() == 3,
             f"{op}: k and v must be 3D (length, num_kv_heads, head_dim)")
    _require(k_cache.dtype == v_cache.dtype == k.dtype == v.dtype,
             f"{op}: k_cache, v_cache, k, v must have the same dtype")
    _require(indices.dtype == torch.int32, f"{op}: indices must be int32")
    _require(k_cache.dtype in _DTYPES, f"{op}: unsupported dtype, must be float16 or bfloat16")
    num_slots, hkv, d = k_cache.shape
    length = indices.shape[0]
    _require(d % 4 == 0, f"{op}: head_dim must be a multiple of 4")
    _require(v_cache.shape == k_cache.shape, f"{op}: v_cache shape must match k_cache")
    _require(tuple(k.shape) == (length, hkv, d) and tuple(v.shape) == (length, hkv, d),
             f"{op}: k and v shape must be (length, num_kv_heads, head_dim)")
    _require(k_cache.is_cuda and all(t.device == k_cache.device for t in (v_cache, indices, k, v)),
             f"{op}: tensors must live on the same CUDA device")
    for t in (k_cache, v_cache, k, v):
        _require(t.stride(2) == 1 and t.stride(1) == d, f"{op}: rows must be dense")
    _require(k.stride(0) == v.stride(0) and k_cache.stride(0) == v_cache.stride(0),
             f"{op}: k/v (and the two caches) must share their row stride")
    _require(indices.is_contiguous(), f"{op}: indices must be contiguous")
    sh = _stream_handle(stream, k_cache.device)
    with _on_device(k_cache.device):
        status = _workspace(256, k_cache.device, sh, "decode")   # dropped rows are reported there
        _lib.check(_lib.lib().msgl_store_kv_cache(
            k_cache.data_ptr(), v_cache.data_ptr(), indices.data_ptr(), k.data_ptr(), v.data_ptr(),
            length, hkv, d, num_slots, k_cache.stride(0), k.stride(0), _DTYPES[k_cache.dtype],
            status.data_ptr(), sh))


def qk_norm_rope_store(q, k, v, q_weight, k_weight, positions, out_loc, k_cache, v_cache, *,
                       rope_base: float, eps: float = 1e-6, rotary_dim: Optional[int] = None,
                       stream=None) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotary embedding of both, and the K/V scatter, in one pass.

    What a Qwen3 attention layer does between its projections and the attention call
    (mini_sglang_mlx/models/qwen3.py:58-68: ``q_norm``, ``k_norm``, ``rope(q)``, ``rope(k)``)
    followed by the store of ``AttnBackend.forward`` (attention/backend.py:117-121).  ``q`` is
    updated in place and returned; the new K rows go to ``k_cache[out_loc]`` normalised and
    rotated, the V rows to ``v_cache[out_loc]`` unchanged.  ``q``, ``k``, ``v`` may be views
    into one fused projection output (dense heads, any token stride).  ``q_weight`` /
    ``k_weight``: (head_dim,) or None to skip that norm.
    """
    op = "qk_norm_rope_store"
    _require(q.dim() == 3 and k.dim() == 3 and v.dim() == 3,
             f"{op}: q must be (n_tokens, num_q_heads, head_dim), k and v (n_tokens, num_kv_heads, head_dim)")
    n, hq, d = q.shape
    hkv = k.shape[1]
    _require(tuple(k.shape) == (n, hkv, d) and tuple(v.shape) == (n, hkv, d),
             f"{op}: k and v shape must be (n_tokens, num_kv_heads, head_dim)")
    _require(q.dtype in _DTYPES and all(t.dtype == q.dtype for t in (k, v, k_cache, v_cache)),
             f"{op}: q, k, v and the caches must share a dtype, float16 or bfloat16")
    for wt in (q_weight, k_weight):
        _require(wt is None or (wt.dtype == q.dtype and tuple(wt.shape) == (d,) and wt.is_contiguous()),
                 f"{op}: a norm weight must be (head_dim,) in the data dtype")
    _require(k_cache.dim() == 3 and tuple(k_cache.shape[1:]) == (hkv, d) and v_cache.shape == k_cache.shape,
             f"{op}: k_cache and v_cache must be (num_pages, num_kv_heads, head_dim)")
    _require(positions.dtype == torch.int32 and out_loc.dtype == torch.int32
             and tuple(positions.shape) == (n,) and tuple(out_loc.shape) == (n,)
             and positions.is_contiguous() and out_loc.is_contiguous(),
             f"{op}: positions and out_loc must be contiguous int32 of n_tokens elements")
    for t in (q, k, v, k_cache, v_cache):
        _require(t.stride(2) == 1 and t.stride(1) == d, f"{op}: rows must be dense")
    _require(k_cache.stride(0) == v_cache.stride(0), f"{op}: the two caches must share their row stride")
    _require(q.is_cuda and all(t.device == q.device for t in (k, v, positions, out_loc, k_cache, v_cache)),
             f"{op}: tensors must live on the same CUDA device")
    rd = d if rotary_dim is None else int(rotary_dim)
    sh = _stream_handle(stream, q.device)
    with _on_device(q.device):
        _lib.check(_lib.lib().msgl_qk_norm_rope_store(
            q.data_ptr(), k.data_ptr(), v.data_ptr(),
            q_weight.data_ptr() if q_weight is not None else None,
            k_weight.data_ptr() if k_weight is not None else None,
            positions.data_ptr(), out_loc.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            n, hq, hkv, d, rd, float(rope_base), float(eps), k_cache.shape[0],
            q.stride(0), k.stride(0), v.stride(0), k_cache.stride(0), _DTYPES[q.dtype], sh))
    return q


def gather_kv_indices(page_table, table_idx, kv_indptr, total_kv: int, *, stream=None):
    """``kv_indices[kv_indptr[b] + t] = page_table[table_idx[b], t]`` for
    ``t < kv_indptr[b+1] - kv_indptr[b]``, in one launch.  Device-side form of the
    per-request loops of AttnBackend.build_*_metadata
    (mini_sglang_mlx/attention/backend.py:239-244, 279-284)."""
    op = "gather_kv_indices"
    _require(page_table.dim() == 2 and page_table.dtype == torch.int32 and page_table.stride(1) == 1,
             f"{op}: page_table must be a 2D int32 tensor with dense rows")
    _require(table_idx.dtype == torch.int32 and kv_indptr.dtype == torch.int32,
             f"{op}: table_idx and kv_indptr must be int32")
    _require(page_table.is_cuda and table_idx.device == page_table.device
             and kv_indptr.device == page_table.device, f"{op}: tensors must be on one CUDA device")
    batch = table_idx.numel()
    _require(kv_indptr.numel() == batch + 1, f"{op}: kv_indptr must have batch+1 entries")
    out = torch.empty(int(total_kv), dtype=torch.int32, device=page_table.device)
    sh = _stream_handle(stream, page_table.device)
    with _on_device(page_table.device):
        status = _workspace(256, page_table.device, sh, "decode")
        _lib.check(_lib.lib().msgl_gather_kv_indices(
            page_table.data_ptr(), page_table.stride(0), table_idx.contiguous().data_ptr(),
            kv_indptr.contiguous().data_ptr(), out.data_ptr(), batch, int(total_kv),
            page_table.shape[0], page_table.shape[1], status.data_ptr(), sh))
    return out


def build_attn_metadata(req_host: torch.Tensor, page_table: torch.Tensor, *, total_q: int, total_kv: int,
                        page_size: int = 1, split_chunk: int = 0, max_kv_splits: int = 32,
                        per_token_ids: bool = True, total_pages: int = None, stream=None):
    """Every index array of a step from the device page table with ONE host-to-device copy and
    ONE launch.  ``req_host``: (3, batch) int32 on the host (pinned for a copy that does not
    block): new tokens, KV lengths, page-table rows.  Returns a dict of int32 device views into
    one buffer: ``qo_indptr``, ``kv_indptr``, ``prefix_lens``, ``num_kv_splits``, ``positions``,
    ``kv_lens``, ``kv_indices`` (or None) and, with ``page_size`` > 1, ``page_indptr`` /
    ``page_indices``.  Device-side form of AttnBackend.build_prefill_metadata /
    build_decode_metadata (mini_sglang_mlx/attention/backend.py:205-307)."""
    op = "build_attn_metadata"
    _require(req_host.dim() == 2 and req_host.shape[0] == 3 and req_host.dtype == torch.int32
             and not req_host.is_cuda and req_host.is_contiguous(),
             f"{op}: req must be a contiguous (3, batch) int32 host tensor")
    _require(page_table.dim() == 2 and page_table.dtype == torch.int32 and page_table.stride(1) == 1
             and page_table.is_cuda, f"{op}: page_table must be a 2D int32 CUDA tensor with dense rows")
    dev = page_table.device
    batch = req_host.shape[1]
    paged = int(page_size) > 1
    if not paged:
        total_pages = 0
    elif total_pages is None:   # (the caller usually knows it: pass it and save the host pass)
        kv = req_host.numpy()[1].astype("int64")
        total_pages = int(((kv + (page_size - 1)) // page_size).sum())
    sizes = dict(req=3 * batch, qo_indptr=batch + 1, kv_indptr=batch + 1, prefix_lens=batch,
                 num_kv_splits=batch, positions=int(total_q),
                 kv_indices=int(total_kv) if per_token_ids else 0,
                 page_indptr=batch + 1 if paged else 0, page_indices=total_pages)
    sh = _stream_handle(stream, dev)
    # the buffer is allocated and filled on the stream the kernel runs on; with the current stream
    # (the usual call) that needs no stream context
    stream_ctx = _NO_CTX if stream is None else torch.cuda.stream(torch.cuda.ExternalStream(sh, device=dev))
    with _on_device(dev), stream_ctx:
        buf = torch.empty(sum(sizes.values()), dtype=torch.int32, device=dev)
        out, off = {}, 0
        for name, n in sizes.items():
            out[name] = buf[off:off + n]
            off += n
        out["req"].copy_(req_host.view(-1), non_blocking=True)
        status = _workspace(256, dev, sh, "decode")
        ptr = lambda name: out[name].data_ptr() if sizes[name] else None  # noqa: E731
        _lib.check(_lib.lib().msgl_build_attn_metadata(
            out["req"].data_ptr(), page_table.data_ptr(), page_table.stride(0), page_table.shape[0],
            page_table.shape[1], batch, int(page_size), int(split_chunk), int(max_kv_splits),
            int(total_q), int(total_kv), total_pages, out["qo_indptr"].data_ptr(),
            out["kv_indptr"].data_ptr(), out["prefix_lens"].data_ptr(), out["num_kv_splits"].data_ptr(),
            ptr("positions"), ptr("kv_indices"), ptr("page_indptr"), ptr("page_indices"),
            status.data_ptr(), sh))
    out["kv_lens"] = out["req"][batch:2 * batch]
    if not per_token_ids:
        out["kv_indices"] = None
    if not paged:
        out["page_indptr"] = out["page_indices"] = None
    return out


def fast_compare_key(a, b) -> int:
    """Length of the common prefix of two 1-D int32/int64 keys held in host memory
    (numpy arrays or CPU tensors).  Signature and checks of the reference op:
    mini-sglang-mlx-kernel/csrc/bindings.cpp:33-35, csrc/fast_compare_key.cpp:9-30."""
    import numpy as np
    op = "fast_compare_key"
    a = a.numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    b = b.numpy() if isinstance(b, torch.Tensor) else np.asarray(b)
    _require(a.ndim == 1 and b.ndim == 1, f"{op}: Both arrays must be 1D.")
    _require(a.flags["C_CONTIGUOUS"] and b.flags["C_CONTIGUOUS"], f"{op}: Both arrays must be contiguous.")
    _require(a.dtype == b.dtype, f"{op}: Both arrays must have the same dtype.")
    _require(a.dtype in (np.int32, np.int64), f"{op}: Arrays must be int32 or int64.")
    n = _lib.lib().msgl_fast_compare_key(a.ctypes.data, b.ctypes.data, a.shape[0], b.shape[0], a.itemsize)
    _require(n >= 0, _lib.last_error())
    return int(n)
