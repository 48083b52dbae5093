"""Seeded synthetic inputs with the shapes of the benchmark configurations.

The reference measures on no dataset; these stand in for a serving trace.
Common rules: Q/K/V i.i.d. N(0,1) in bf16, ``sm_scale = 1/sqrt(head_dim)``,
page size 16, a sequence of L tokens owns ``ceil(L/16)`` pages drawn without
replacement from a random permutation of the pool, the slot of token t is
``page*16 + t%16`` (the reference itself hard-wires one token per page,
mini_sglang_mlx/engine/engine.py:103, so a slot id is what it calls a page
id), index arrays are int32.

Also here: the algorithmic byte / flop counts of a workload (each needed byte
counted once) that the roofline fractions are computed from.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

PAGE_SIZE = 16


@dataclass
class Workload:
    name: str
    kind: str                       # "decode" | "prefill"
    hq: int
    hkv: int
    head_dim: int
    q: torch.Tensor
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    kv_indptr: torch.Tensor
    kv_indices: torch.Tensor
    kv_lens: List[int]
    page_table: torch.Tensor        # (batch, max_pages) int32 page ids, -1 padded
    sm_scale: float
    # decode
    num_kv_splits: Optional[torch.Tensor] = None
    max_kv_splits: int = 32
    # prefill
    qo_indptr: Optional[torch.Tensor] = None
    prefix_lens: Optional[torch.Tensor] = None
    q_lens: List[int] = field(default_factory=list)
    max_len_extend: int = 0
    is_cross_attention: bool = False
    sliding_window_size: int = 0
    seed: int = 0

    @property
    def batch(self) -> int:
        return len(self.kv_lens)

    def page_csr(self):
        """(page_indptr, page_indices, kv_lens) int32 on the workload's device: the page-granular
        form of ``kv_indptr`` / ``kv_indices`` (one id per 16-token page)."""
        need = [(l + PAGE_SIZE - 1) // PAGE_SIZE for l in self.kv_lens]
        dev = self.q.device
        table = self.page_table
        parts = [table[b, :n] for b, n in enumerate(need)]
        idx = torch.cat(parts).contiguous() if parts else torch.zeros(0, dtype=torch.int32, device=dev)
        return (_indptr(need).to(dev), idx.to(torch.int32),
                torch.tensor(self.kv_lens, dtype=torch.int32, device=dev))

    # ---- algorithmic work: K+V of the visible keys once per KV head, Q and O once,
    # one int32 index per visible key token
    def visible_keys_per_seq(self) -> List[int]:
        if self.kind == "decode":
            return list(self.kv_lens)
        out = []
        for L, tq in zip(self.kv_lens, self.q_lens):
            prefix = L - tq
            lo = max(0, prefix - self.sliding_window_size + 1) if self.sliding_window_size > 0 else 0
            out.append(L - lo)
        return out

    index: str = "token"            # "token": one int32 id per KV token; "page": one per 16-token page

    def algorithmic_bytes(self) -> int:
        vis = sum(self.visible_keys_per_seq())
        kv = 2 * vis * self.hkv * self.head_dim * 2
        qo = 2 * self.q.shape[0] * self.hq * self.head_dim * 2
        ids = vis if self.index == "token" else sum((v + PAGE_SIZE - 1) // PAGE_SIZE
                                                     for v in self.visible_keys_per_seq())
        return kv + qo + 4 * ids

    def algorithmic_flops(self) -> int:
        if self.kind == "decode":
            pairs = sum(self.kv_lens)
        else:
            pairs = 0
            W = self.sliding_window_size
            for L, tq in zip(self.kv_lens, self.q_lens):
                prefix = L - tq
                for p in range(tq):
                    pos = prefix + p
                    hi = L - 1 if self.is_cross_attention else min(pos, L - 1)
                    lo = max(0, pos - W + 1) if W > 0 else 0
                    pairs += max(0, hi - lo + 1)
        return 4 * self.head_dim * self.hq * pairs


def reference_num_kv_splits(kv_lens: List[int], max_kv_splits: int = 32) -> List[int]:
    """Split rule of the reference backend (mini_sglang_mlx/attention/backend.py:304-307)."""
    return [min(max_kv_splits, max(1, (l + 127) // 128)) for l in kv_lens]


def _alloc_pages(kv_lens: List[int], num_pages: int, gen: torch.Generator):
    need = [(l + PAGE_SIZE - 1) // PAGE_SIZE for l in kv_lens]
    if sum(need) > num_pages:
        raise ValueError(f"pool of {num_pages} pages is too small for {sum(need)} pages")
    perm = torch.randperm(num_pages, generator=gen)
    max_pages = max(need) if need else 0
    table = torch.full((len(kv_lens), max(max_pages, 1)), -1, dtype=torch.int32)
    off = 0
    for b, n in enumerate(need):
        table[b, :n] = perm[off:off + n].to(torch.int32)
        off += n
    return table


def slots_from_page_table(table: torch.Tensor, kv_lens: List[int]) -> torch.Tensor:
    """Per-token slot ids (int32, CSR order): slot = page*16 + t%16."""
    parts = []
    for b, L in enumerate(kv_lens):
        t = torch.arange(L, dtype=torch.int64)
        parts.append((table[b, t // PAGE_SIZE].to(torch.int64) * PAGE_SIZE + t % PAGE_SIZE).to(torch.int32))
    return torch.cat(parts) if parts else torch.zeros(0, dtype=torch.int32)


def _randn_bf16(shape, device, seed: int) -> torch.Tensor:
    """N(0,1) in bf16 generated on ``device`` in bounded chunks."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    flat = out.view(-1)
    step = 1 << 28
    for s in range(0, flat.numel(), step):
        n = min(step, flat.numel() - s)
        flat[s:s + n] = torch.randn(n, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    return out


def _indptr(lens: List[int]) -> torch.Tensor:
    return torch.tensor([0] + list(torch.tensor(lens, dtype=torch.int64).cumsum(0).tolist()),
                        dtype=torch.int32) if lens else torch.zeros(1, dtype=torch.int32)


def _log_uniform(lo: int, hi: int, n: int, gen: torch.Generator) -> List[int]:
    u = torch.rand(n, generator=gen, dtype=torch.float64)
    return [int(round(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo))))) for x in u]


def make_decode(name: str, *, hq: int, hkv: int, kv_lens: List[int], num_pages: int, seed: int,
                device, head_dim: int = 128, max_kv_splits: int = 32,
                num_kv_splits: Optional[List[int]] = None) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    table = _alloc_pages(kv_lens, num_pages, gen)
    slots = slots_from_page_table(table, kv_lens)
    num_slots = num_pages * PAGE_SIZE
    dev = torch.device(device)
    splits = num_kv_splits if num_kv_splits is not None else reference_num_kv_splits(kv_lens, max_kv_splits)
    return Workload(
        name=name, kind="decode", hq=hq, hkv=hkv, head_dim=head_dim,
        q=_randn_bf16((len(kv_lens), hq, head_dim), dev, seed + 1),
        k_cache=_randn_bf16((num_slots, hkv, head_dim), dev, seed + 2),
        v_cache=_randn_bf16((num_slots, hkv, head_dim), dev, seed + 3),
        kv_indptr=_indptr(kv_lens).to(dev), kv_indices=slots.to(dev), kv_lens=list(kv_lens),
        page_table=table.to(dev), sm_scale=1.0 / math.sqrt(head_dim),
        num_kv_splits=torch.tensor(splits, dtype=torch.int32, device=dev),
        max_kv_splits=max_kv_splits, seed=seed)


def make_prefill(name: str, *, hq: int, hkv: int, q_lens: List[int], prefix_lens: List[int],
                 num_pages: int, seed: int, device, head_dim: int = 128,
                 is_cross_attention: bool = False, sliding_window_size: int = 0) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    kv_lens = [p + t for p, t in zip(prefix_lens, q_lens)]
    table = _alloc_pages(kv_lens, num_pages, gen)
    slots = slots_from_page_table(table, kv_lens)
    num_slots = num_pages * PAGE_SIZE
    dev = torch.device(device)
    return Workload(
        name=name, kind="prefill", hq=hq, hkv=hkv, head_dim=head_dim,
        q=_randn_bf16((sum(q_lens), hq, head_dim), dev, seed + 1),
        k_cache=_randn_bf16((num_slots, hkv, head_dim), dev, seed + 2),
        v_cache=_randn_bf16((num_slots, hkv, head_dim), dev, seed + 3),
        kv_indptr=_indptr(kv_lens).to(dev), kv_indices=slots.to(dev), kv_lens=kv_lens,
        page_table=table.to(dev), sm_scale=1.0 / math.sqrt(head_dim),
        qo_indptr=_indptr(q_lens).to(dev),
        prefix_lens=torch.tensor(prefix_lens, dtype=torch.int32, device=dev),
        q_lens=list(q_lens), max_len_extend=max(q_lens) if q_lens else 0,
        is_cross_attention=is_cross_attention, sliding_window_size=sliding_window_size, seed=seed)


# ------------------------------------------------------------------ the benchmark configurations
def cfg1_decode(seed: int = 101, device="cuda", batch: int = 8) -> Workload:
    """Decode, Qwen3-0.6B shape: Hq16/Hkv8, B=8, L ~ U{256..2048}, 4096-page pool."""
    gen = torch.Generator().manual_seed(seed)
    kv_lens = torch.randint(256, 2049, (batch,), generator=gen).tolist()
    return make_decode("cfg1_decode_qwen3_0.6b", hq=16, hkv=8, kv_lens=kv_lens, num_pages=4096,
                       seed=seed, device=device)


def cfg2_prefill(seed: int = 202, device="cuda", batch: int = 4, chunk: int = 512,
                 max_prefix: int = 4096, num_pages: int = 32768) -> Workload:
    """Chunked prefill, Qwen3-8B shape: Hq32/Hkv8, B=4, prefix ~ U{0..4096} + 512-token chunk, causal."""
    gen = torch.Generator().manual_seed(seed)
    prefix = torch.randint(0, max_prefix + 1, (batch,), generator=gen).tolist()
    return make_prefill("cfg2_chunked_prefill_qwen3_8b", hq=32, hkv=8, q_lens=[chunk] * batch,
                        prefix_lens=prefix, num_pages=num_pages, seed=seed, device=device)


def cfg3_window_block(seed: int = 303, device="cuda", batch: int = 16, block: int = 16,
                      kv_len: int = 8192, window: int = 4096, cross: bool = False) -> Workload:
    """Sliding-window block for a draft layer: Hq32/Hkv8, B=16, 16 query tokens over KV 8192
    (prefix 8176 + the block), window 4096, causal inside the block unless ``cross``."""
    pages = batch * ((kv_len + PAGE_SIZE - 1) // PAGE_SIZE)
    return make_prefill("cfg3_sliding_window_block", hq=32, hkv=8, q_lens=[block] * batch,
                        prefix_lens=[kv_len - block] * batch, num_pages=2 * pages, seed=seed,
                        device=device, is_cross_attention=cross, sliding_window_size=window)


def cfg4_verify(seed: int = 404, device="cuda", batch: int = 32, q_tokens: int = 8,
                lo: int = 1024, hi: int = 32768) -> Workload:
    """Speculative verify, Qwen3-30B-A3B attention shape: Hq32/Hkv4, B=32, 8 query tokens,
    prior KV length log-uniform in [1024, 32768], causal."""
    gen = torch.Generator().manual_seed(seed)
    prior = _log_uniform(lo, hi, batch, gen)
    pages = sum((p + q_tokens + PAGE_SIZE - 1) // PAGE_SIZE for p in prior)
    return make_prefill("cfg4_spec_verify_qwen3_30b_a3b", hq=32, hkv=4, q_lens=[q_tokens] * batch,
                        prefix_lens=prior, num_pages=pages + pages // 8 + 16, seed=seed, device=device)


def cfg5a_decode(seed: int = 505, device="cuda", batch: int = 256, lo: int = 4096,
                 hi: int = 131072, num_kv_splits: Optional[List[int]] = None,
                 max_kv_splits: int = 32) -> Workload:
    """Long-context decode, Qwen3-8B shape: Hq32/Hkv8, B=256, L log-uniform in [4096, 131072]."""
    gen = torch.Generator().manual_seed(seed)
    kv_lens = _log_uniform(lo, hi, batch, gen)
    pages = sum((l + PAGE_SIZE - 1) // PAGE_SIZE for l in kv_lens)
    return make_decode("cfg5a_long_context_decode_qwen3_8b", hq=32, hkv=8, kv_lens=kv_lens,
                       num_pages=pages + pages // 64 + 16, seed=seed, device=device,
                       num_kv_splits=num_kv_splits, max_kv_splits=max_kv_splits)


def d256_prefill_point(hkv: int, hq: int, q_len: int, prefix: int = 0, seed: int = 707,
                       device="cuda") -> Workload:
    """head_dim 256, one sequence of ``q_len`` new tokens after ``prefix`` cached ones, causal:
    the shapes of the reference's own prefill sweep (head configurations (kv, q) = (2, 16),
    (4, 16), (4, 24), (2, 32); mini-sglang-mlx-kernel/test_and_bench/paged_prefill_attention.py:20-26, 329-331)."""
    pages = (q_len + prefix + PAGE_SIZE - 1) // PAGE_SIZE
    return make_prefill(f"d256_prefill_kv{hkv}_q{hq}_t{q_len}_p{prefix}", hq=hq, hkv=hkv,
                        q_lens=[q_len], prefix_lens=[prefix], num_pages=pages + pages // 4 + 16,
                        seed=seed + q_len + prefix, device=device, head_dim=256)


def d256_decode_point(hkv: int, hq: int, kv_len: int, batch: int = 1, seed: int = 808,
                      device="cuda") -> Workload:
    """head_dim 256 decode over ``batch`` sequences of ``kv_len`` tokens: the shapes of the
    reference's own decode sweep (single sequences and uniform batches;
    mini-sglang-mlx-kernel/test_and_bench/paged_decode_attention.py:18-23, 241-257)."""
    pages = batch * ((kv_len + PAGE_SIZE - 1) // PAGE_SIZE)
    return make_decode(f"d256_decode_kv{hkv}_q{hq}_l{kv_len}_b{batch}", hq=hq, hkv=hkv,
                       kv_lens=[kv_len] * batch, num_pages=pages + pages // 4 + 16,
                       seed=seed + kv_len + batch, device=device, head_dim=256)


CFG5B_CHUNKS = (128, 256, 512, 1024, 2048, 4096)
CFG5B_PREFIXES = (1024, 2048, 4096, 8192, 16384, 32768)


def cfg5b_prefill_point(chunk: int, prefix: int, seed: int = 606, device="cuda") -> Workload:
    """One point of the 6x6 prefill grid: Hq32/Hkv8, B=1, ``chunk`` new tokens after a cached
    prefix of ``prefix`` tokens, causal."""
    pages = (chunk + prefix + PAGE_SIZE - 1) // PAGE_SIZE
    w = make_prefill(f"cfg5b_prefill_c{chunk}_p{prefix}", hq=32, hkv=8, q_lens=[chunk],
                     prefix_lens=[prefix], num_pages=pages + pages // 4 + 16,
                     seed=seed + chunk + prefix, device=device)
    return w
