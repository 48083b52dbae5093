"""Attention with the output gate fused into the final write: out = attention * sigmoid(gate)
(the array op after the attention call of the reference's Qwen3.5 layer,
mini_sglang_mlx/models/qwen3_5.py:91-110), against the oracle chain attention -> round to the
16-bit type -> times sigmoid(gate) rounded to the 16-bit type.  Every final-write site is
covered: decode merge, prefill direct epilogue (both CTA shapes), prefill kv-split merge."""
import math

import pytest
import torch

from oracle import paged_attention_oracle as O
from tests.helpers import assert_close_to_oracle
from tests.test_prefill_gpu import make_inputs

pytestmark = pytest.mark.gpu


def _gated(ref, gate):
    dt = gate.dtype
    return (ref.to(dt).float() * torch.sigmoid(gate.float()).to(dt).float()).to(dt)


def _same_up_to_one_rounding(out, ref):
    """The kernel gates its own rounded output; against the same chain on the host only the
    sigmoid's last bit can differ (hardware exp against torch's): two 16-bit ulps at most."""
    assert torch.allclose(out.cpu().float(), ref.float(), rtol=2 ** -7, atol=1e-30)


@pytest.mark.parametrize("q_lens,prefixes,d", [([300, 17], [100, 700], 128),    # two-sub-tile shape, direct write
                                               ([8, 8], [9000, 3000], 128),      # verify shape: kv split + merge
                                               ([16], [40], 128),                # one-sub-tile shape, direct write
                                               ([130, 5], [260, 0], 256)])       # head_dim 256
def test_prefill_with_gate(q_lens, prefixes, d):
    from mini_sglang_mlx_b200 import paged_prefill_attention
    x = make_inputs(q_lens, prefixes, 2, 8, seed=11, d=d)
    gate = (torch.randn(x["q"].shape, generator=torch.Generator().manual_seed(5)) * 2).bfloat16()
    out = paged_prefill_attention(x["q"], x["k_cache"], x["v_cache"], x["qo_indptr"], x["kv_indptr"],
                                  x["kv_indices"], x["prefix_lens"], 1 / math.sqrt(d), x["max_len_extend"],
                                  gate=gate.cuda())
    ref = O.paged_prefill_attention_oracle(x["q"], x["k_cache"], x["v_cache"], x["qo_indptr"], x["kv_indptr"],
                                           x["kv_indices"], x["prefix_lens"], 1 / math.sqrt(d))
    assert_close_to_oracle(out, _gated(ref.cpu(), gate).float(), f"gated prefill {q_lens}")
    plain = paged_prefill_attention(x["q"], x["k_cache"], x["v_cache"], x["qo_indptr"], x["kv_indptr"],
                                    x["kv_indices"], x["prefix_lens"], 1 / math.sqrt(d), x["max_len_extend"])
    _same_up_to_one_rounding(out, _gated(plain.cpu().float(), gate))


@pytest.mark.parametrize("d", [128, 256])
def test_decode_with_gate(d):
    from mini_sglang_mlx_b200 import paged_decode_attention
    x = make_inputs([1, 1, 1], [1500, 63, 4097], 4, 16, seed=8, d=d)
    splits = torch.tensor([4, 1, 8], dtype=torch.int32).cuda()
    gate = torch.randn(x["q"].shape, generator=torch.Generator().manual_seed(6)).bfloat16()
    args = (x["q"], x["k_cache"], x["v_cache"], x["kv_indptr"], x["kv_indices"], splits, 1 / math.sqrt(d), 8)
    out = paged_decode_attention(*args, gate=gate.cuda())
    plain = paged_decode_attention(*args)
    _same_up_to_one_rounding(out, _gated(plain.cpu().float(), gate))
    with pytest.raises(RuntimeError, match="gate must match q"):
        paged_decode_attention(*args, gate=gate.cuda()[:2])
