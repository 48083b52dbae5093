"""Fused q/k RMSNorm + RoPE + K/V scatter against the CPU restatement of the reference's
separate array ops (mini_sglang_mlx/models/qwen3.py:58-68 + attention/backend.py:117-121).

Tolerance: the kernel and the oracle share the fp32 formulas and both round to the 16-bit
type after the norm and after the rotation; they differ in the fp32 evaluation of
rsqrt / sin / cos, so a result may land on the neighbouring 16-bit value: max abs error
<= 2e-2 and mean abs error <= 2e-3 (the attention path's bar), V rows and untouched
slots bit-exact."""
import pytest
import torch

from oracle.qk_norm_rope_oracle import qk_norm_rope_store_oracle

pytestmark = pytest.mark.gpu


def _case(n, hq, hkv, dtype, seed, max_pos, num_slots=4096, fused_qkv=False, d=128):
    g = torch.Generator().manual_seed(seed)
    if fused_qkv:
        qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).to(dtype)
        q = qkv[:, : hq * d].view(n, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
    else:
        qkv = None
        q = (torch.randn(n, hq, d, generator=g) * 3).to(dtype)
        k = (torch.randn(n, hkv, d, generator=g) * 0.5).to(dtype)
        v = torch.randn(n, hkv, d, generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    pos = torch.randint(0, max_pos, (n,), generator=g, dtype=torch.int32)
    loc = torch.randperm(num_slots, generator=g)[:n].int()
    kc = torch.randn(num_slots, hkv, d, generator=g).to(dtype)
    vc = torch.randn(num_slots, hkv, d, generator=g).to(dtype)
    return qkv, q, k, v, qw, kw, pos, loc, kc, vc


def _check(out, ref, what):
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max().item() <= 2e-2 * max(1.0, ref.float().abs().max().item()), f"{what}: max {err.max().item()}"
    assert err.mean().item() <= 2e-3, f"{what}: mean {err.mean().item()}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,hq,hkv,d,rd,max_pos", [
    (1, 16, 8, 128, 128, 10), (37, 32, 8, 128, 128, 40000), (300, 32, 4, 128, 128, 131072),
    (64, 16, 8, 128, 64, 5000), (33, 7, 3, 128, 32, 900),
    # head_dim 256: the whole head, half of it, and a quarter (the reference's Qwen3.5 layers)
    (40, 16, 4, 256, 256, 30000), (9, 8, 2, 256, 128, 70000), (130, 24, 4, 256, 64, 100000), (5, 3, 1, 256, 64, 17)])
def test_fused_step_matches_the_separate_ops(dtype, n, hq, hkv, d, rd, max_pos):
    from mini_sglang_mlx_b200 import qk_norm_rope_store
    _, q, k, v, qw, kw, pos, loc, kc, vc = _case(n, hq, hkv, dtype, seed=n + rd, max_pos=max_pos, d=d)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = qk_norm_rope_store_oracle(q, k, v, qw, kw, pos, loc, kc_ref, vc_ref,
                                      rope_base=1e6, eps=1e-6, rotary_dim=rd)
    dev = "cuda"
    qd, kcd, vcd = q.to(dev), kc.to(dev), vc.to(dev)
    out = qk_norm_rope_store(qd, k.to(dev), v.to(dev), qw.to(dev), kw.to(dev), pos.to(dev), loc.to(dev),
                             kcd, vcd, rope_base=1e6, eps=1e-6, rotary_dim=rd)
    assert out.data_ptr() == qd.data_ptr()
    _check(out, q_ref, "q")
    _check(kcd, kc_ref, "k_cache")
    assert torch.equal(vcd.cpu(), vc_ref), "v rows and untouched slots must be bit-exact"
    untouched = torch.ones(kc.shape[0], dtype=torch.bool)
    untouched[loc.long()] = False
    assert torch.equal(kcd.cpu()[untouched], kc[untouched])


def test_views_into_a_fused_projection_and_no_norm_weights():
    from mini_sglang_mlx_b200 import qk_norm_rope_store
    qkv, q, k, v, _, _, pos, loc, kc, vc = _case(50, 32, 8, torch.bfloat16, 5, 9000, fused_qkv=True)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = qk_norm_rope_store_oracle(q, k, v, None, None, pos, loc, kc_ref, vc_ref,
                                      rope_base=10000.0, eps=1e-6, rotary_dim=128)
    qkv_d = qkv.cuda()
    hq, hkv, d = 32, 8, 128
    qd = qkv_d[:, : hq * d].view(50, hq, d)
    kd = qkv_d[:, hq * d:(hq + hkv) * d].view(50, hkv, d)
    vd = qkv_d[:, (hq + hkv) * d:].view(50, hkv, d)
    kcd, vcd = kc.cuda(), vc.cuda()
    qk_norm_rope_store(qd, kd, vd, None, None, pos.cuda(), loc.cuda(), kcd, vcd, rope_base=10000.0)
    _check(qd, q_ref, "q view")
    _check(kcd, kc_ref, "k_cache")
    assert torch.equal(vcd.cpu(), vc_ref)
    assert torch.equal(kd.cpu(), k), "the k input is not modified"


def test_out_of_range_slots_are_dropped_and_bad_arguments_rejected():
    from mini_sglang_mlx_b200 import qk_norm_rope_store
    _, q, k, v, qw, kw, pos, loc, kc, vc = _case(8, 16, 8, torch.bfloat16, 9, 100, num_slots=64)
    loc[3] = 64
    loc[5] = -1
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = qk_norm_rope_store_oracle(q, k, v, qw, kw, pos, loc, kc_ref, vc_ref,
                                      rope_base=1e6, eps=1e-6, rotary_dim=128)
    kcd, vcd = kc.cuda(), vc.cuda()
    out = qk_norm_rope_store(q.cuda(), k.cuda(), v.cuda(), qw.cuda(), kw.cuda(), pos.cuda(), loc.cuda(),
                             kcd, vcd, rope_base=1e6)
    _check(out, q_ref, "q")
    _check(kcd, kc_ref, "k_cache")
    assert torch.equal(vcd.cpu(), vc_ref)
    with pytest.raises(RuntimeError, match="rotary_dim must be head_dim, head_dim/2 or head_dim/4"):
        qk_norm_rope_store(q.cuda(), k.cuda(), v.cuda(), None, None, pos.cuda(), loc.cuda(), kcd, vcd,
                           rope_base=1e6, rotary_dim=48)
    with pytest.raises(RuntimeError, match="positions and out_loc"):
        qk_norm_rope_store(q.cuda(), k.cuda(), v.cuda(), None, None, pos.cuda().long(), loc.cuda(), kcd, vcd,
                           rope_base=1e6)


def test_fused_step_then_attention_equals_the_unfused_layer():
    """q/k/v -> fused step -> paged prefill, against the oracle chain norm -> rope -> store -> attention."""
    from mini_sglang_mlx_b200 import paged_prefill_attention, qk_norm_rope_store
    from oracle import paged_attention_oracle as O
    from tests.helpers import assert_close_to_oracle
    n, hq, hkv, d = 200, 32, 8, 128
    _, q, k, v, qw, kw, _, loc, kc, vc = _case(n, hq, hkv, torch.bfloat16, 21, 1, num_slots=1024)
    pos = torch.arange(n, dtype=torch.int32)
    kc.zero_(); vc.zero_()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = qk_norm_rope_store_oracle(q, k, v, qw, kw, pos, loc, kc_ref, vc_ref,
                                      rope_base=1e6, eps=1e-6, rotary_dim=128)
    meta = [torch.tensor([0, n], dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32), loc,
            torch.tensor([0], dtype=torch.int32)]
    ref = O.paged_prefill_attention_oracle(q_ref, kc_ref, vc_ref, *meta, d ** -0.5)
    kcd, vcd = kc.cuda(), vc.cuda()
    qd = qk_norm_rope_store(q.cuda(), k.cuda(), v.cuda(), qw.cuda(), kw.cuda(), pos.cuda(), loc.cuda(),
                            kcd, vcd, rope_base=1e6)
    out = paged_prefill_attention(qd, kcd, vcd, *[m.cuda() for m in meta], d ** -0.5, n)
    assert_close_to_oracle(out, ref, "fused step + prefill")


def test_backend_forward_from_projections_equals_norm_rope_then_forward():
    """AttnBackend.forward_from_projections (fused step + attention) against the oracle chain
    norm -> rope -> AttnBackend.forward, for a chunked prefill with a cached prefix and a decode step."""
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    from oracle.qk_norm_rope_oracle import rms_norm_oracle, rope_oracle
    from tests.helpers import assert_close_to_oracle

    class Cfg:
        head_dim, num_kv_heads, num_qo_heads = 128, 8, 32

    g = torch.Generator().manual_seed(31)
    pools = [MHAKVCache(8, 1, 128, 2049, torch.bfloat16) for _ in range(2)]
    table = torch.randperm(2048, generator=g)[: 4 * 512].view(4, 512).int().cuda()
    fused, plain = AttnBackend(Cfg, pools[0], table), AttnBackend(Cfg, pools[1], table)
    qw = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16()
    reqs = [Req(table_idx=2, cached_len=0, device_len=130), Req(table_idx=0, cached_len=0, device_len=33)]
    for phase in (BatchPhase.PREFILL, BatchPhase.DECODE):
        n = sum(r.extend_len for r in reqs)
        q = (torch.randn(n, 32, 128, generator=g) * 2).bfloat16()
        k = torch.randn(n, 8, 128, generator=g).bfloat16()
        v = torch.randn(n, 8, 128, generator=g).bfloat16()
        out_loc = torch.cat([table[r.table_idx, r.cached_len:r.device_len] for r in reqs])
        batch = Batch(reqs=reqs, phase=phase, out_loc=out_loc)
        fused.prepare_metadata(batch)
        pos = batch.attn_metadata.positions.cpu()
        out_f = fused.forward_from_projections(q.cuda(), k.cuda(), v.cuda(), 0, batch, q_norm_weight=qw.cuda(),
                                               k_norm_weight=kw.cuda(), rope_base=1e6)
        qn = rope_oracle(rms_norm_oracle(q, qw, 1e-6), pos, 1e6, 128)
        kn = rope_oracle(rms_norm_oracle(k, kw, 1e-6), pos, 1e6, 128)
        out_p = plain.forward(qn.cuda(), kn.cuda(), v.cuda(), 0, batch)
        assert_close_to_oracle(out_f, out_p.float().cpu(), f"fused layer {phase}")
        for r in reqs:
            r.complete_one()


def test_fused_step_into_a_pool_beyond_4_gib_per_tensor():
    """K/V rows scattered to slots whose byte offset needs more than 32 bits."""
    from mini_sglang_mlx_b200 import qk_norm_rope_store
    n, hq, hkv, d, S = 6, 16, 8, 128, 2_300_000
    _, q, k, v, qw, kw, pos, _, _, _ = _case(n, hq, hkv, torch.bfloat16, seed=3, max_pos=50000, num_slots=64)
    loc = torch.tensor([S - 1, 2_097_152, 2_097_999, 2_250_000, 0, 1_048_576], dtype=torch.int32)
    small_k = torch.zeros(8, hkv, d, dtype=torch.bfloat16)       # the oracle scatters into a dense pool
    kc_ref, vc_ref = small_k.clone(), small_k.clone()
    q_ref = qk_norm_rope_store_oracle(q, k, v, qw, kw, pos, torch.arange(n, dtype=torch.int32), kc_ref, vc_ref,
                                      rope_base=1e6, eps=1e-6, rotary_dim=d)
    kcd = torch.zeros(S, hkv, d, dtype=torch.bfloat16, device="cuda")
    vcd = torch.zeros_like(kcd)
    out = qk_norm_rope_store(q.cuda(), k.cuda(), v.cuda(), qw.cuda(), kw.cuda(), pos.cuda(), loc.cuda(),
                             kcd, vcd, rope_base=1e6, eps=1e-6, rotary_dim=d)
    torch.cuda.synchronize()
    _check(out, q_ref, "q")
    rows = loc.long().cuda()
    _check(kcd[rows], kc_ref[:n], "k rows")
    assert torch.equal(vcd[rows].cpu(), vc_ref[:n])
    assert int((kcd != 0).any(dim=(1, 2)).sum()) == n and int((vcd != 0).any(dim=(1, 2)).sum()) == n
