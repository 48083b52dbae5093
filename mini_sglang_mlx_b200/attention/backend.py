"""Attention backend: CSR metadata from the page table, K/V store, dispatch.

Mirror of the reference's ``AttnBackend``
(mini_sglang_mlx/attention/backend.py:64-307): same class, method and field
names and the same meaning of every argument, over CUDA ``torch.Tensor``.
Differences, all inside the boundary:

* every index array of a step (``qo_indptr``, ``kv_indptr``, ``kv_indices``,
  ``prefix_lens``, ``positions``, ``num_kv_splits``) comes from ONE launch over the
  device-resident page table after ONE host-to-device copy of the per-request
  lengths and table rows (pinned staging), instead of per-request loops and several
  small copies on the host (reference lines 205-307).
* ``page_size`` > 1 (the reference has one token per page,
  mini_sglang_mlx/engine/engine.py:103): the table rows hold page-structured slots
  (``CacheManager(page_size=...)``), the metadata also carries one id per page
  (``page_indptr`` / ``page_indices`` / ``kv_lens``) and, when the page size is a
  multiple of 16, attention runs through the page-granular operators whose kernels
  fetch K/V as TMA boxes.
* ``num_kv_splits`` is chosen for a 148-SM part from the batch's total work
  (``compute_num_kv_splits``); ``policy="reference"`` keeps the reference rule
  ``min(32, max(1, ceil(L/128)))`` (lines 304-307).  The result of the decode
  op does not depend on the choice beyond fp32 rounding.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import _lib
from ..kernel import (build_attn_metadata, paged_decode_attention, paged_decode_attention_p16,
                      paged_prefill_attention, paged_prefill_attention_p16, qk_norm_rope_store)

MAX_KV_SPLITS = 32


@dataclass
class BaseAttnMetadata:
    positions: torch.Tensor

    def get_last_indices(self, bs: int) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class PrefillMetadata(BaseAttnMetadata):
    qo_indptr: torch.Tensor     # (batch + 1,) int32
    kv_indptr: torch.Tensor     # (batch + 1,) int32
    kv_indices: torch.Tensor    # (total_kv,) int32 slot ids
    prefix_lens: torch.Tensor   # (batch,) int32
    max_len_extend: int
    # page-granular form (None with one token per page)
    page_indptr: Optional[torch.Tensor] = None   # (batch + 1,) int32
    page_indices: Optional[torch.Tensor] = None  # (total_pages,) int32 page ids
    kv_lens: Optional[torch.Tensor] = None       # (batch,) int32
    page_size: int = 1

    def get_last_indices(self, bs: int) -> torch.Tensor:
        return self.qo_indptr[1:1 + bs] - 1


@dataclass
class DecodeMetadata(BaseAttnMetadata):
    kv_indptr: torch.Tensor     # (batch + 1,) int32
    kv_indices: torch.Tensor    # (total_kv,) int32 slot ids
    num_kv_splits: torch.Tensor  # (batch,) int32
    max_kv_splits: int
    page_indptr: Optional[torch.Tensor] = None
    page_indices: Optional[torch.Tensor] = None
    kv_lens: Optional[torch.Tensor] = None
    page_size: int = 1

    def get_last_indices(self, bs: int) -> torch.Tensor:
        return torch.arange(bs, dtype=torch.int32, device=self.kv_indptr.device)


AttnMetadata = PrefillMetadata | DecodeMetadata


def compute_num_kv_splits(kv_lens: Sequence[int], num_kv_heads: int, *, sm_count: int = 148,
                          max_kv_splits: int = MAX_KV_SPLITS, policy: str = "b200") -> List[int]:
    """Per-sequence split count of the decode op.

    ``reference``: ``min(max, max(1, ceil(L/128)))`` (reference lines 304-307).
    ``b200``: one split per ``chunk`` tokens (``split_chunk_tokens``).
    """
    if policy == "reference":
        return [min(max_kv_splits, max(1, (l + 127) // 128)) for l in kv_lens]
    chunk = split_chunk_tokens(sum(kv_lens), num_kv_heads, sm_count=sm_count, batch=len(kv_lens))
    return [min(max_kv_splits, max(1, -(-l // chunk))) for l in kv_lens]


def split_chunk_tokens(total_kv: int, num_kv_heads: int, *, sm_count: int = 148, batch: int = 0,
                       policy: str = "b200") -> int:
    """Tokens per split of the decode op for a batch with ``total_kv`` KV tokens.

    ``b200``: the batch's ``total_kv * num_kv_heads`` token-heads spread over about 16 CTAs per
    SM, clamped to [256, 4096] tokens: enough CTAs to fill the SMs, small enough that a long
    sequence does not leave a tail.  A small batch that would then need a little more than one
    wave of CTAs (two are resident per SM) gets the chunk that makes it exactly one: a CTA of
    such a batch is a chain of memory latencies, and a second, partial wave doubles it."""
    if policy == "reference":
        return 128
    chunk = -(-total_kv * num_kv_heads // (sm_count * 16))
    chunk = min(4096, max(256, chunk))
    slots = 2 * sm_count
    ctas = (total_kv // chunk + batch) * num_kv_heads          # upper bound with this chunk
    room = slots // num_kv_heads - batch                        # split slots per head in one wave
    if batch > 0 and room > 0 and slots < ctas <= 2 * slots:
        chunk = min(4096, max(chunk, -(-total_kv // room)))
    return -(-chunk // 64) * 64


class AttnBackend:
    """Paged attention backend for B200 using the msgl C-ABI operators."""

    def __init__(self, config, kvcache, page_table: torch.Tensor, *,
                 split_policy: str = "b200", page_size: int = 1) -> None:
        self.config = config
        self.kvcache = kvcache
        self.page_table = page_table      # (rows, max_seq_len) int32 per-token slot ids, on device
        self.sm_scale = 1.0 / math.sqrt(config.head_dim)
        self.split_policy = split_policy
        self.page_size = int(page_size)
        # the page-granular operators are the fast path when their kernels can fetch whole
        # 16-row boxes; other page sizes keep the per-token ids
        self._paged_ops = self.page_size % 16 == 0
        self._sm_count: Optional[int] = None
        self._staging: List[torch.Tensor] = []        # pinned (3, capacity) int32 buffers, in turn
        self._staging_events: List[torch.cuda.Event] = []
        self._staging_next = 0

    # ------------------------------------------------------------------ forward
    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_id: int, batch, *,
                is_cross_attention: bool = False, sliding_window_size: int = 0,
                gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Write this step's K/V rows at ``batch.out_loc`` and run paged attention.

        q ``[N, Hq, D]``, k/v ``[N, Hkv, D]``.  The mask flags compose as in the
        reference (lines 97-132): causal / full / causal+window /
        bidirectional+window; the decode path accepts neither.  ``gate`` (same shape as
        q, an addition to the reference signature): the result is multiplied by
        ``sigmoid(gate)`` in the kernel's final write (the reference's Qwen3.5 layer does it
        as an array op afterwards, models/qwen3_5.py:110).
        """
        assert sliding_window_size >= 0, (
            f"sliding_window_size must be >= 0, got {sliding_window_size}")
        metadata = batch.attn_metadata
        self.kvcache.store_kv(k, v, batch.out_loc, layer_id)
        k_cache = self.kvcache.k_cache(layer_id)
        v_cache = self.kvcache.v_cache(layer_id)
        return self._attend(q, k_cache, v_cache, metadata, is_cross_attention, sliding_window_size, gate)

    def _attend(self, q, k_cache, v_cache, metadata, is_cross_attention: bool,
                sliding_window_size: int, gate=None) -> torch.Tensor:
        paged = self._paged_ops and metadata.page_indices is not None
        if isinstance(metadata, PrefillMetadata):
            if paged:
                return paged_prefill_attention_p16(
                    q, k_cache, v_cache, metadata.qo_indptr, metadata.page_indptr, metadata.page_indices,
                    metadata.kv_lens, metadata.prefix_lens, sm_scale=self.sm_scale,
                    max_len_extend=metadata.max_len_extend, page_size=metadata.page_size,
                    is_cross_attention=is_cross_attention, sliding_window_size=sliding_window_size,
                    gate=gate)
            return paged_prefill_attention(
                q, k_cache, v_cache, metadata.qo_indptr, metadata.kv_indptr, metadata.kv_indices,
                metadata.prefix_lens, sm_scale=self.sm_scale, max_len_extend=metadata.max_len_extend,
                is_cross_attention=is_cross_attention, sliding_window_size=sliding_window_size, gate=gate)
        assert isinstance(metadata, DecodeMetadata)
        assert not is_cross_attention and sliding_window_size == 0, (
            "is_cross_attention / sliding_window_size are only supported on the prefill path.")
        if paged:
            return paged_decode_attention_p16(
                q, k_cache, v_cache, metadata.page_indptr, metadata.page_indices, metadata.kv_lens,
                metadata.num_kv_splits, sm_scale=self.sm_scale, max_kv_splits=metadata.max_kv_splits,
                page_size=metadata.page_size, gate=gate)
        return paged_decode_attention(
            q, k_cache, v_cache, metadata.kv_indptr, metadata.kv_indices, metadata.num_kv_splits,
            sm_scale=self.sm_scale, max_kv_splits=metadata.max_kv_splits, gate=gate)

    def forward_from_projections(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_id: int,
                                 batch, *, q_norm_weight, k_norm_weight, rope_base: float,
                                 rms_norm_eps: float = 1e-6, rotary_dim: Optional[int] = None,
                                 is_cross_attention: bool = False, sliding_window_size: int = 0,
                                 gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``forward`` for a layer that hands over its raw projections: the per-head q/k
        RMSNorm, the rotary embedding at ``batch.attn_metadata.positions`` and the K/V store
        run as one pass (``qk_norm_rope_store``; q is updated in place), then paged attention.

        Equivalent to the reference layer's ``q_norm``, ``k_norm``, ``rope``, ``rope`` followed by
        ``AttnBackend.forward`` (mini_sglang_mlx/models/qwen3.py:58-68)."""
        assert sliding_window_size >= 0, (
            f"sliding_window_size must be >= 0, got {sliding_window_size}")
        metadata = batch.attn_metadata
        k_cache = self.kvcache.k_cache(layer_id)
        v_cache = self.kvcache.v_cache(layer_id)
        qk_norm_rope_store(q, k, v, q_norm_weight, k_norm_weight, metadata.positions, batch.out_loc,
                           k_cache, v_cache, rope_base=rope_base, eps=rms_norm_eps, rotary_dim=rotary_dim)
        return self._attend(q, k_cache, v_cache, metadata, is_cross_attention, sliding_window_size, gate)

    def store_kv_only(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor,
                      layer_id: int) -> None:
        """Write K/V into the pool without running attention (reference lines 174-196)."""
        self.kvcache.store_kv(k, v, out_loc, layer_id)

    # ------------------------------------------------------------------ metadata
    def prepare_metadata(self, batch) -> None:
        reqs = batch.padded_reqs
        if batch.is_prefill:
            batch.attn_metadata = self.build_prefill_metadata(reqs)
        else:
            batch.attn_metadata = self.build_decode_metadata(reqs)

    def _stage(self, extend_lens: Sequence[int], kv_lens: Sequence[int], rows: Sequence[int]):
        """The per-request numbers of a step as a pinned, contiguous (3, batch) int32 tensor and
        the event to record behind the copy that reads it.  Four buffers take turns; one is
        written again only after the copy that last read it has finished."""
        n = len(kv_lens)
        if not self._staging or self._staging[0].numel() < 3 * n:
            cap = max(64, 1 << max(n - 1, 0).bit_length())
            self._staging = [torch.empty(3 * cap, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._staging_np = [t.numpy() for t in self._staging]   # same memory, cheap row writes
            self._staging_events = [torch.cuda.Event() for _ in range(4)]
            self._staging_next = 0
        k = self._staging_next
        self._staging_next = (k + 1) % len(self._staging)
        self._staging_events[k].synchronize()
        req = self._staging[k][: 3 * n].view(3, n)
        rows_np = self._staging_np[k][: 3 * n].reshape(3, n)
        rows_np[0] = extend_lens
        rows_np[1] = kv_lens
        rows_np[2] = rows
        return req, self._staging_events[k]

    def _index_arrays(self, reqs, extend_lens: Sequence[int], kv_lens: Sequence[int], split_chunk: int):
        req, event = self._stage(extend_lens, kv_lens, [r.table_idx for r in reqs])
        ps = self.page_size if self._paged_ops else 1
        md = build_attn_metadata(req, self.page_table, total_q=sum(extend_lens), total_kv=sum(kv_lens),
                                 page_size=ps, split_chunk=split_chunk, max_kv_splits=MAX_KV_SPLITS,
                                 per_token_ids=not self._paged_ops,
                                 total_pages=sum((l + ps - 1) // ps for l in kv_lens) if ps > 1 else 0)
        event.record()
        return md

    def build_prefill_metadata(self, reqs, *, extend_lens: Optional[List[int]] = None,
                               kv_lens: Optional[List[int]] = None,
                               positions: Optional[torch.Tensor] = None) -> PrefillMetadata:
        """Reference lines 205-254; ``extend_lens`` / ``kv_lens`` overrides serve a
        virtual extend window such as a K+1-token verify."""
        if extend_lens is None:
            extend_lens = [req.extend_len for req in reqs]
        if kv_lens is None:
            kv_lens = [req.device_len for req in reqs]
        md = self._index_arrays(reqs, extend_lens, kv_lens, 0)
        return PrefillMetadata(positions=md["positions"] if positions is None else positions,
                               qo_indptr=md["qo_indptr"], kv_indptr=md["kv_indptr"],
                               kv_indices=md["kv_indices"], prefix_lens=md["prefix_lens"],
                               max_len_extend=max(extend_lens), page_indptr=md["page_indptr"],
                               page_indices=md["page_indices"], kv_lens=md["kv_lens"],
                               page_size=self.page_size if self._paged_ops else 1)

    def build_decode_metadata(self, reqs, *, kv_lens: Optional[List[int]] = None,
                              positions: Optional[torch.Tensor] = None) -> DecodeMetadata:
        """Reference lines 256-293."""
        if kv_lens is None:
            kv_lens = [req.device_len for req in reqs]
        if self._sm_count is None:
            with torch.cuda.device(self.page_table.device):
                self._sm_count = max(1, _lib.lib().msgl_device_sm_count())
        chunk = split_chunk_tokens(sum(kv_lens), self.config.num_kv_heads, sm_count=self._sm_count,
                                   batch=len(kv_lens), policy=self.split_policy)
        # "new tokens" of a decode row = everything behind what the request has cached, so that
        # the kernel's prefix_lens are the reference's positions (req.cached_len, line 276)
        extend = [max(1, min(kv_lens[i], kv_lens[i] - reqs[i].cached_len)) for i in range(len(reqs))]
        md = self._index_arrays(reqs, extend, kv_lens, chunk)
        # the split dimension of the launch grid: what the longest sequence needs, not the cap
        # (CTAs of split slots no sequence uses would only start, look up a length and leave)
        # (the reference policy keeps the reference's constant, backend.py:293)
        max_splits = MAX_KV_SPLITS
        if self.split_policy != "reference" and kv_lens:
            max_splits = min(MAX_KV_SPLITS, max(1, -(-max(kv_lens) // chunk)))
        return DecodeMetadata(positions=md["prefix_lens"] if positions is None else positions,
                              kv_indptr=md["kv_indptr"], kv_indices=md["kv_indices"],
                              num_kv_splits=md["num_kv_splits"], max_kv_splits=max_splits,
                              page_indptr=md["page_indptr"], page_indices=md["page_indices"],
                              kv_lens=md["kv_lens"], page_size=self.page_size if self._paged_ops else 1)
