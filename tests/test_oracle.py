"""The oracle against the reference's known answers and against an
independent attention routine (CPU only)."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import paged_attention_oracle as O
from tests.helpers import build_kat_inputs, load_mask_kats

KATS = load_mask_kats()


@pytest.mark.parametrize("case", KATS, ids=[c["name"] for c in KATS])
def test_oracle_matches_reference_mask_known_answers(case):
    d = build_kat_inputs(case)
    v_cache = torch.zeros_like(d["k_cache"])
    k_cache = d["k_cache"].clone()
    if case["slots"] is None:
        v_cache[: d["kv_len"]] = d["v_rows"]
    else:  # the reference case writes the rows through store_kv_cache first
        O.store_kv_cache_oracle(k_cache, v_cache, d["kv_indices"],
                                torch.zeros_like(d["v_rows"]), d["v_rows"])
    out = O.paged_prefill_attention_oracle(
        d["q"], k_cache, v_cache, d["qo_indptr"], d["kv_indptr"], d["kv_indices"],
        d["prefix_lens"], d["sm_scale"], is_cross_attention=case["is_cross_attention"],
        sliding_window_size=case["sliding_window_size"])
    actual = out[:, 0, : d["kv_len"]].numpy()
    np.testing.assert_allclose(actual, np.asarray(case["expected_weights"], dtype=np.float32),
                               rtol=case["rtol"], atol=case["atol"])


@pytest.mark.parametrize("case", KATS, ids=[c["name"] for c in KATS])
def test_loop_and_vectorised_mask_agree(case):
    w = O.expected_weights(case["q_len"], case["prefix_len"],
                           is_cross_attention=case["is_cross_attention"],
                           sliding_window_size=case["sliding_window_size"])
    np.testing.assert_allclose(w, np.asarray(case["expected_weights"], dtype=np.float32), atol=1e-7)
    vis = O.visibility_mask(case["q_len"], case["q_len"] + case["prefix_len"], case["prefix_len"],
                            is_cross_attention=case["is_cross_attention"],
                            sliding_window_size=case["sliding_window_size"]).numpy()
    assert ((w > 0) == vis).all()


@pytest.mark.parametrize("cross,window", [(False, 0), (True, 0), (False, 7), (True, 9)])
def test_prefill_oracle_matches_torch_sdpa(cross, window):
    torch.manual_seed(3)
    hq, hkv, d = 8, 2, 128
    tq, pre = [3, 17, 1], [0, 21, 40]
    L = [a + b for a, b in zip(tq, pre)]
    S = sum(L) + 5
    kc = torch.randn(S, hkv, d).bfloat16()
    vc = torch.randn(S, hkv, d).bfloat16()
    q = torch.randn(sum(tq), hq, d).bfloat16()
    slots = torch.randperm(S)[: sum(L)].int()
    qo = torch.from_numpy(O.build_indptr(tq))
    kvp = torch.from_numpy(O.build_indptr(L))
    out = O.paged_prefill_attention_oracle(q, kc, vc, qo, kvp, slots,
                                           torch.tensor(pre, dtype=torch.int32), 1 / math.sqrt(d),
                                           is_cross_attention=cross, sliding_window_size=window)
    for b in range(len(tq)):
        rows = slots[kvp[b]:kvp[b + 1]].long()
        k = kc[rows].float().permute(1, 0, 2).repeat_interleave(hq // hkv, 0)[None]
        v = vc[rows].float().permute(1, 0, 2).repeat_interleave(hq // hkv, 0)[None]
        qq = q[qo[b]:qo[b + 1]].float().permute(1, 0, 2)[None]
        m = O.visibility_mask(tq[b], L[b], pre[b], is_cross_attention=cross, sliding_window_size=window)
        ref = F.scaled_dot_product_attention(qq, k, v, attn_mask=m, scale=1 / math.sqrt(d))[0]
        torch.testing.assert_close(out[qo[b]:qo[b + 1]], ref.permute(1, 0, 2), atol=2e-6, rtol=1e-5)


def test_decode_oracle_equals_prefill_oracle_with_one_query():
    torch.manual_seed(5)
    hq, hkv, d = 4, 2, 128
    L = [1, 33, 130]
    S = sum(L)
    kc, vc = torch.randn(S, hkv, d).bfloat16(), torch.randn(S, hkv, d).bfloat16()
    q = torch.randn(len(L), hq, d).bfloat16()
    slots = torch.randperm(S).int()
    kvp = torch.from_numpy(O.build_indptr(L))
    dec = O.paged_decode_attention_oracle(q, kc, vc, kvp, slots, 0.1)
    pre = O.paged_prefill_attention_oracle(q, kc, vc, torch.arange(len(L) + 1, dtype=torch.int32), kvp,
                                           slots, torch.tensor([l - 1 for l in L], dtype=torch.int32), 0.1)
    torch.testing.assert_close(dec, pre, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("lens", [[1], [237, 809], [128, 129, 4097]])
def test_split_kv_merge_equals_unsplit(lens):
    torch.manual_seed(7)
    hq, hkv, d = 4, 2, 128
    S = sum(lens)
    kc, vc = torch.randn(S, hkv, d).bfloat16(), torch.randn(S, hkv, d).bfloat16()
    q = torch.randn(len(lens), hq, d).bfloat16()
    slots = torch.randperm(S).int()
    kvp = torch.from_numpy(O.build_indptr(lens))
    splits = torch.from_numpy(O.compute_num_kv_splits(lens))
    a = O.split_kv_decode_oracle(q, kc, vc, kvp, slots, splits, 1 / math.sqrt(d))
    b = O.paged_decode_attention_oracle(q, kc, vc, kvp, slots, 1 / math.sqrt(d))
    torch.testing.assert_close(a, b, atol=2e-6, rtol=1e-5)


def test_split_ranges_follow_the_reference_rule():
    # ceil(ceil(L/splits)/32)*32 tokens per split, empty splits skipped
    assert O.decode_split_ranges(4097, 32) == [(i * 160, min(4097, (i + 1) * 160)) for i in range(26)]
    assert O.decode_split_ranges(1, 1) == [(0, 1)]
    assert O.decode_split_ranges(0, 1) == []
    assert list(O.compute_num_kv_splits([1, 128, 129, 5000])) == [1, 1, 2, 32]


def test_empty_and_fully_masked_rows_are_zero():
    hq, hkv, d = 2, 1, 128
    kc = torch.randn(4, hkv, d).bfloat16()
    q = torch.randn(2, hq, d).bfloat16()
    # sequence 0 has no keys; sequence 1 has 2 keys but an inconsistent prefix (-5): row sees nothing
    out = O.paged_prefill_attention_oracle(
        q, kc, kc, torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([0, 0, 2], dtype=torch.int32),
        torch.tensor([1, 2], dtype=torch.int32), torch.tensor([0, -5], dtype=torch.int32), 1.0)
    assert torch.count_nonzero(out) == 0


def test_norm_and_rope_restatements_match_the_transformers_implementations():
    """The q/k RMSNorm and the non-interleaved RoPE of oracle/qk_norm_rope_oracle.py against the
    independent implementations of the same two formulas that ship with transformers."""
    tq = pytest.importorskip("transformers.models.qwen3.modeling_qwen3")
    from oracle.qk_norm_rope_oracle import rms_norm_oracle, rope_oracle
    g = torch.Generator().manual_seed(0)
    x = torch.randn(11, 8, 128, generator=g)
    pos = torch.randint(0, 5000, (11,), generator=g)
    base = 1e6
    inv = base ** (-torch.arange(0, 128, 2, dtype=torch.float32) / 128)
    fr = pos.float()[:, None] * inv[None, :]
    emb = torch.cat([fr, fr], -1)
    xh = x.permute(1, 0, 2)[None]                      # (batch 1, heads, tokens, d)
    out, _ = tq.apply_rotary_pos_emb(xh, xh, emb.cos()[None], emb.sin()[None])
    assert (out[0].permute(1, 0, 2) - rope_oracle(x, pos, base, 128)).abs().max().item() < 1e-5
    norm = tq.Qwen3RMSNorm(128, eps=1e-6)
    norm.weight.data = 1 + 0.1 * torch.randn(128, generator=g)
    assert (norm(x) - rms_norm_oracle(x, norm.weight.data, 1e-6)).abs().max().item() < 1e-6
    # partial rotary: the upper elements pass through
    half = rope_oracle(x, pos, base, 64)
    assert torch.equal(half[..., 64:], x[..., 64:])
