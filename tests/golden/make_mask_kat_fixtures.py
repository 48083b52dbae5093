"""Writes ``mask_kats.json``: the analytic known-answer cases of the
reference's mask tests
(mini-sglang-mlx-kernel/test_and_bench/test_paged_prefill_attention_masks.py:97-158).

Each case is Q = 0, K = 0 (so every visible key gets the same weight) and V
one-hot at column = key position, so an output row *is* the row of attention
weights.  The expected weights are computed here with the reference's own
rule (its ``_expected_weights``, lines 59-71, restated as a loop); no kernel
and no third-party attention routine is involved, so the fixture can be made
on any machine: ``python tests/golden/make_mask_kat_fixtures.py``.
"""
import json
from pathlib import Path

CASES = [
    # name, q_len, prefix_len, is_cross_attention, sliding_window_size, slot ids (None = identity)
    ("default_prefill_remains_causal", 4, 0, False, 0, None),
    ("full_attention_is_unmasked", 4, 0, True, 0, None),
    ("sliding_causal_window", 4, 0, False, 2, None),
    ("sliding_causal_window_crosses_prefix_boundary", 4, 4, False, 5, None),
    ("bidirectional_windowed_over_prefix", 4, 4, True, 5, None),
    ("bidirectional_window_clips_prefix_only", 2, 6, True, 3, None),
    # store_kv_cache writes rows at slots [3,1,4,2] of a 5-slot pool, prefill reads them back
    ("store_kv_cache_writes_are_reachable_by_prefill", 4, 0, False, 0, [3, 1, 4, 2]),
]


def expected(q_len, prefix_len, cross, window):
    kv_len = prefix_len + q_len
    rows = []
    for p in range(q_len):
        pos = prefix_len + p
        attend = [k for k in range(kv_len)
                  if (window == 0 or k >= pos - window + 1) and (cross or k <= pos)]
        rows.append([1.0 / len(attend) if k in attend else 0.0 for k in range(kv_len)])
    return rows


def main():
    out = []
    for name, q_len, prefix, cross, window, slots in CASES:
        out.append(dict(name=name, q_len=q_len, prefix_len=prefix, is_cross_attention=cross,
                        sliding_window_size=window, slots=slots, head_dim=128,
                        rtol=1e-3, atol=1e-3, expected_weights=expected(q_len, prefix, cross, window)))
    path = Path(__file__).with_name("mask_kats.json")
    path.write_text(json.dumps(out, indent=1))
    print(f"wrote {path} ({len(out)} cases)")


if __name__ == "__main__":
    main()
