"""fp32 gather-then-SDPA oracle for the paged attention operators (CPU).

TEST INFRASTRUCTURE ONLY — never imported by the product package.

What it restates, and from where (paths inside the reference project):

* decode: per sequence, gather ``k_cache[kv_indices[s:e]]`` and run plain
  softmax attention with no mask —
  ``mini-sglang-mlx-kernel/test_and_bench/paged_decode_attention.py:98-131``
  (``run_mlx_sdpa``).
* prefill: per sequence, gather, build the boolean visibility mask and run
  softmax attention —
  ``mini-sglang-mlx-kernel/test_and_bench/paged_prefill_attention.py:114-180``;
  the four-mode mask is the truth function of
  ``mini-sglang-mlx-kernel/test_and_bench/test_paged_prefill_attention_masks.py:59-71``
  and of the kernel's ``apply_attention_mask``
  (``mini-sglang-mlx-kernel/csrc/paged_prefill_attention.metal:324-350``).
* the two-stage split-KV decode with log-sum-exp merge —
  ``mini-sglang-mlx-kernel/csrc/paged_decode_attention.metal:356-363, 494-505,
  554-585`` — restated to show that it equals the unsplit result.
* ``store_kv_cache`` scatter —
  ``mini-sglang-mlx-kernel/csrc/store_kv_cache.metal:7-31``.
* the CSR metadata builders and the split rule —
  ``mini_sglang_mlx/attention/backend.py:205-307``.

The softmax-attention arithmetic itself lives in a third-party dependency of
the reference, ``mlx`` (``mx.fast.scaled_dot_product_attention``; requirement
``mlx>=0.31.2``, no lock file), which is not installable here; it is the
standard ``softmax(scale * Q K^T + mask) V`` with grouped-query head sharing
and is restated directly.  Pinning: the mask semantics and slot addressing are
pinned by the reference's analytic known-answer cases (restated in
``tests/golden/make_mask_kat_fixtures.py`` and checked by
``tests/test_oracle.py``); the attention arithmetic is cross-checked against
``torch.nn.functional.scaled_dot_product_attention``.  No output of the
reference's own kernels could be produced on this machine (they need
macOS/Metal).

All math is float32 on inputs upcast from the caller's tensors; GQA maps
``kv_head = q_head // (Hq // Hkv)``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

MAX_KV_SPLITS = 32  # mini_sglang_mlx/attention/backend.py:15


# --------------------------------------------------------------------------- masks
def expected_weights(q_len: int, prefix_len: int, *, is_cross_attention: bool = False,
                     sliding_window_size: int = 0) -> np.ndarray:
    """Attention weights of the all-zero-score known-answer cases: uniform over
    the visible keys of each query row.  Loop form of
    test_paged_prefill_attention_masks.py:59-71."""
    kv_len = prefix_len + q_len
    w = np.zeros((q_len, kv_len), dtype=np.float32)
    for p in range(q_len):
        pos = prefix_len + p
        attend = [
            kpos for kpos in range(kv_len)
            if (sliding_window_size == 0 or kpos >= pos - sliding_window_size + 1)
            and (is_cross_attention or kpos <= pos)
        ]
        w[p, attend] = 1.0 / len(attend)
    return w


def visibility_mask(q_len: int, kv_len: int, prefix_len: int, *, is_cross_attention: bool = False,
                    sliding_window_size: int = 0, q_offset: int = 0) -> torch.Tensor:
    """Boolean (q_len, kv_len): key t visible to query row q_offset + i.
    Vectorised form of the truth function above
    (csrc/paged_prefill_attention.metal:324-350)."""
    pos = prefix_len + q_offset + torch.arange(q_len).unsqueeze(1)
    kpos = torch.arange(kv_len).unsqueeze(0)
    vis = torch.ones(q_len, kv_len, dtype=torch.bool)
    if not is_cross_attention:
        vis &= kpos <= pos
    if sliding_window_size > 0:
        vis &= kpos >= pos - sliding_window_size + 1
    return vis


# --------------------------------------------------------------------------- attention core
def _attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
            mask: Optional[torch.Tensor]) -> torch.Tensor:
    """q (Tq,Hq,D), k/v (L,Hkv,D) float32 -> (Tq,Hq,D).  Rows with no visible
    key give zeros (csrc/paged_prefill_attention.metal:627-630)."""
    tq, hq, d = q.shape
    L, hkv, _ = k.shape
    g = hq // hkv
    if L == 0 or tq == 0:
        return torch.zeros(tq, hq, d, dtype=torch.float32)
    qh = q.permute(1, 0, 2).reshape(hkv, g * tq, d)          # (Hkv, G*Tq, D), head-major rows
    kh = k.permute(1, 0, 2)                                   # (Hkv, L, D)
    vh = v.permute(1, 0, 2)
    s = torch.bmm(qh, kh.transpose(1, 2)) * scale             # (Hkv, G*Tq, L)
    if mask is not None:
        m = mask.unsqueeze(0).repeat(g, 1, 1).reshape(g * tq, L)  # row order: (g, token)
        s = s.masked_fill(~m.unsqueeze(0), float("-inf"))
    smax = s.max(dim=-1, keepdim=True).values
    smax = torch.where(torch.isinf(smax), torch.zeros_like(smax), smax)
    p = torch.exp(s - smax)
    den = p.sum(dim=-1, keepdim=True)
    o = torch.bmm(p, vh)
    o = torch.where(den > 0, o / den.clamp_min(1e-38), torch.zeros_like(o))
    return o.reshape(hkv, g, tq, d).reshape(hq, tq, d).permute(1, 0, 2).contiguous()


def paged_decode_attention_oracle(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale: float,
                                  seqs: Optional[Sequence[int]] = None) -> torch.Tensor:
    """(batch, Hq, D) float32; ``seqs`` restricts the computation to some
    sequences (the other rows are left zero)."""
    q = q.detach().cpu()
    indptr = kv_indptr.detach().cpu().to(torch.int64)
    idx = kv_indices.detach().cpu().to(torch.int64)
    batch, hq, d = q.shape
    out = torch.zeros(batch, hq, d, dtype=torch.float32)
    for b in (range(batch) if seqs is None else seqs):
        s, e = int(indptr[b]), int(indptr[b + 1])
        rows = idx[s:e]
        k = k_cache[rows.to(k_cache.device)].detach().cpu().float()
        v = v_cache[rows.to(v_cache.device)].detach().cpu().float()
        out[b] = _attend(q[b:b + 1].float(), k, v, sm_scale, None)[0]
    return out


def paged_prefill_attention_oracle(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices,
                                   prefix_lens, sm_scale: float, *, is_cross_attention: bool = False,
                                   sliding_window_size: int = 0,
                                   seqs: Optional[Sequence[int]] = None,
                                   q_block: int = 1024) -> torch.Tensor:
    """(total_q, Hq, D) float32.  Long query chunks are processed in blocks of
    ``q_block`` rows to bound the score matrix."""
    q = q.detach().cpu()
    qo = qo_indptr.detach().cpu().to(torch.int64)
    indptr = kv_indptr.detach().cpu().to(torch.int64)
    idx = kv_indices.detach().cpu().to(torch.int64)
    pre = prefix_lens.detach().cpu().to(torch.int64)
    total_q, hq, d = q.shape
    out = torch.zeros(total_q, hq, d, dtype=torch.float32)
    batch = qo.numel() - 1
    for b in (range(batch) if seqs is None else seqs):
        qs, qe = int(qo[b]), int(qo[b + 1])
        s, e = int(indptr[b]), int(indptr[b + 1])
        L = e - s
        rows = idx[s:e]
        k = k_cache[rows.to(k_cache.device)].detach().cpu().float()
        v = v_cache[rows.to(v_cache.device)].detach().cpu().float()
        for q0 in range(qs, qe, q_block):
            q1 = min(qe, q0 + q_block)
            mask = visibility_mask(q1 - q0, L, int(pre[b]), is_cross_attention=is_cross_attention,
                                   sliding_window_size=sliding_window_size, q_offset=q0 - qs)
            out[q0:q1] = _attend(q[q0:q1].float(), k, v, sm_scale, mask)
    return out


# --------------------------------------------------------------------------- split-KV restatement
def decode_split_ranges(L: int, splits: int, round_to: int = 32) -> List[Tuple[int, int]]:
    """Token ranges of the active splits of a sequence of length L
    (csrc/paged_decode_attention.metal:356-363): length per split is
    ceil(ceil(L/splits)/32)*32; empty splits are skipped."""
    if L <= 0:
        return []
    per = math.ceil(math.ceil(L / splits) / round_to) * round_to
    return [(s * per, min(L, (s + 1) * per)) for s in range(splits) if s * per < L]


def split_kv_decode_oracle(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits,
                           sm_scale: float) -> torch.Tensor:
    """Two-stage decode: normalised partial O and lse = max + ln(sum) per
    split, then the log-sum-exp merge (csrc/paged_decode_attention.metal:494-505,
    554-585).  Equal to ``paged_decode_attention_oracle`` up to fp32 rounding."""
    q = q.detach().cpu().float()
    indptr = kv_indptr.detach().cpu().to(torch.int64)
    idx = kv_indices.detach().cpu().to(torch.int64)
    splits = num_kv_splits.detach().cpu().to(torch.int64)
    batch, hq, d = q.shape
    hkv = k_cache.shape[1]
    g = hq // hkv
    out = torch.zeros(batch, hq, d, dtype=torch.float32)
    for b in range(batch):
        s0, e0 = int(indptr[b]), int(indptr[b + 1])
        rows = idx[s0:e0]
        k = k_cache[rows].detach().cpu().float()
        v = v_cache[rows].detach().cpu().float()
        parts, lses = [], []
        for (a, z) in decode_split_ranges(e0 - s0, int(splits[b])):
            kk = k[a:z].permute(1, 0, 2).repeat_interleave(g, dim=0)       # (Hq, n, D)
            vv = v[a:z].permute(1, 0, 2).repeat_interleave(g, dim=0)
            sc = torch.einsum("hd,hnd->hn", q[b], kk) * sm_scale
            m = sc.max(dim=-1, keepdim=True).values
            p = torch.exp(sc - m)
            den = p.sum(dim=-1, keepdim=True)
            parts.append(torch.einsum("hn,hnd->hd", p, vv) / den)
            lses.append((m + torch.log(den)).squeeze(-1))
        if not parts:
            continue
        lse = torch.stack(lses)                                             # (S, Hq)
        w = torch.exp(lse - lse.max(dim=0, keepdim=True).values)
        out[b] = (w.unsqueeze(-1) * torch.stack(parts)).sum(0) / w.sum(0).unsqueeze(-1)
    return out


# --------------------------------------------------------------------------- pool write side
def store_kv_cache_oracle(k_cache, v_cache, indices, k, v) -> None:
    """In place, in row order (later rows win on duplicate slots):
    csrc/store_kv_cache.metal:7-31."""
    for r in range(int(indices.shape[0])):
        pos = int(indices[r])
        k_cache[pos] = k[r]
        v_cache[pos] = v[r]


# --------------------------------------------------------------------------- metadata
def build_indptr(lens: Sequence[int]) -> np.ndarray:
    """mini_sglang_mlx/attention/backend.py:299-301."""
    return np.cumsum(np.asarray([0] + list(lens), dtype=np.int32), dtype=np.int32)


def compute_num_kv_splits(kv_lens: Sequence[int]) -> np.ndarray:
    """mini_sglang_mlx/attention/backend.py:304-307."""
    return np.asarray([min(MAX_KV_SPLITS, max(1, (l + 127) // 128)) for l in kv_lens], dtype=np.int32)


def build_prefill_metadata_oracle(page_table: np.ndarray, table_idx: Sequence[int],
                                  extend_lens: Sequence[int], kv_lens: Sequence[int]):
    """mini_sglang_mlx/attention/backend.py:205-254: returns positions,
    qo_indptr, kv_indptr, kv_indices, prefix_lens, max_len_extend."""
    cached = [kv_lens[i] - extend_lens[i] for i in range(len(kv_lens))]
    positions = np.concatenate(
        [np.arange(cached[i], kv_lens[i], dtype=np.int32) for i in range(len(kv_lens))]
        or [np.zeros(0, dtype=np.int32)])
    kv_indices = np.concatenate(
        [page_table[table_idx[i], : kv_lens[i]] for i in range(len(kv_lens))]
        or [np.zeros(0, dtype=np.int32)]).astype(np.int32)
    return (positions, build_indptr(extend_lens), build_indptr(kv_lens), kv_indices,
            np.asarray(cached, dtype=np.int32), max(extend_lens))


def build_decode_metadata_oracle(page_table: np.ndarray, table_idx: Sequence[int],
                                 kv_lens: Sequence[int], cached_lens: Sequence[int]):
    """mini_sglang_mlx/attention/backend.py:256-293: returns positions,
    kv_indptr, kv_indices, num_kv_splits, max_kv_splits."""
    kv_indices = np.concatenate(
        [page_table[table_idx[i], : kv_lens[i]] for i in range(len(kv_lens))]
        or [np.zeros(0, dtype=np.int32)]).astype(np.int32)
    return (np.asarray(cached_lens, dtype=np.int32), build_indptr(kv_lens), kv_indices,
            compute_num_kv_splits(kv_lens), MAX_KV_SPLITS)
