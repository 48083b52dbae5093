"""CPU restatement of the step in front of the attention op (TEST INFRASTRUCTURE ONLY).

The reference composes it from array ops (mini_sglang_mlx/models/qwen3.py:58-68):
``nn.RMSNorm`` on the per-head q and k, ``RotaryEmbedding`` (mini_sglang_mlx/layers/
rotary_embedding.py:17-20: ``nn.RoPE(rotary_dim, base=base)`` with ``offset=positions``,
i.e. the non-interleaved layout) on both, then ``AttnBackend.forward`` scatters K/V
(attention/backend.py:117-121).  ``nn.RMSNorm`` and ``nn.RoPE`` live in the third-party
``mlx`` package (requirement ``mlx>=0.31.2``), which is absent here: parity unpinned
against mlx itself.  Their published definitions are restated below (fp32 arithmetic, one
rounding to the 16-bit type after each op, as each op materialises an array), and
``tests/test_oracle.py`` checks the restatement against the independent implementations
of the same two formulas in the ``transformers`` package (Qwen3RMSNorm, rotate-half RoPE).
"""
from __future__ import annotations

import torch


def rms_norm_oracle(x: torch.Tensor, weight, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight over the last axis, fp32, rounded to x.dtype."""
    x32 = x.float()
    y = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def rope_oracle(x: torch.Tensor, positions: torch.Tensor, base: float, rotary_dim: int) -> torch.Tensor:
    """x: (n, heads, d).  Pairs (i, i + rotary_dim/2), angle = position * base^(-2i/rotary_dim);
    elements past rotary_dim pass through."""
    half = rotary_dim // 2
    freqs = base ** (-torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim)
    theta = positions.to(torch.float32)[:, None] * freqs[None, :]          # fp32 product, as mlx does
    cos = torch.cos(theta.double()).float()[:, None, :]
    sin = torch.sin(theta.double()).float()[:, None, :]
    x32 = x.float()
    x1, x2, rest = x32[..., :half], x32[..., half:rotary_dim], x32[..., rotary_dim:]
    out = torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos, rest], dim=-1)
    return out.to(x.dtype)


def qk_norm_rope_store_oracle(q, k, v, q_weight, k_weight, positions, out_loc, k_cache, v_cache, *,
                              rope_base: float, eps: float, rotary_dim: int) -> torch.Tensor:
    """Returns the processed q; writes the processed k and the raw v into the caches at
    out_loc (tokens with an out-of-range slot are dropped).  A weight of None means that the
    layer has no norm on that input (the norm is skipped, not run with unit weights)."""
    qn = rope_oracle(q if q_weight is None else rms_norm_oracle(q, q_weight, eps), positions, rope_base, rotary_dim)
    kn = rope_oracle(k if k_weight is None else rms_norm_oracle(k, k_weight, eps), positions, rope_base, rotary_dim)
    ok = (out_loc >= 0) & (out_loc < k_cache.shape[0])
    idx = out_loc[ok].long()
    k_cache[idx] = kn[ok]
    v_cache[idx] = v[ok]
    return qn
