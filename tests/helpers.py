"""Shared helpers of the test-suite: tolerances, KAT builders, comparisons."""
import json
import math
from pathlib import Path

import numpy as np
import torch

# Tolerances of the port against the fp32 oracle (bf16 outputs, fp32 accumulation).
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_mask_kats():
    return json.loads((GOLDEN / "mask_kats.json").read_text())


def build_kat_inputs(case, device="cpu", dtype=torch.bfloat16):
    """Inputs of one known-answer case: Q = 0, K = 0, V one-hot at column = key position."""
    q_len, prefix, d = case["q_len"], case["prefix_len"], case["head_dim"]
    kv_len = prefix + q_len
    slots = case["slots"]
    num_slots = kv_len if slots is None else max(slots) + 1
    q = torch.zeros(q_len, 1, d, dtype=dtype, device=device)
    k_cache = torch.zeros(num_slots, 1, d, dtype=dtype, device=device)
    v_rows = torch.zeros(kv_len, 1, d, dtype=dtype, device=device)
    for pos in range(kv_len):
        v_rows[pos, 0, pos] = 1.0
    idx = torch.arange(kv_len, dtype=torch.int32, device=device) if slots is None else \
        torch.tensor(slots, dtype=torch.int32, device=device)
    return dict(
        q=q, k_cache=k_cache, v_rows=v_rows, kv_indices=idx, num_slots=num_slots,
        qo_indptr=torch.tensor([0, q_len], dtype=torch.int32, device=device),
        kv_indptr=torch.tensor([0, kv_len], dtype=torch.int32, device=device),
        prefix_lens=torch.tensor([prefix], dtype=torch.int32, device=device),
        sm_scale=1.0 / math.sqrt(d), kv_len=kv_len)


def assert_close_to_oracle(out: torch.Tensor, ref: torch.Tensor, what: str = "",
                           max_tol: float = MAX_ABS_TOL, mean_tol: float = MEAN_ABS_TOL):
    out = out.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(out).all(), f"{what}: non-finite values in the output"
    diff = (out - ref).abs()
    mx = float(diff.max()) if diff.numel() else 0.0
    mean = float(diff.mean()) if diff.numel() else 0.0
    assert mx <= max_tol and mean <= mean_tol, \
        f"{what}: max abs err {mx:.4g} (tol {max_tol}), mean abs err {mean:.4g} (tol {mean_tol})"
    return mx, mean
