"""The factored no-RoPE form (reference: ``launch_factored_attention``,
src/e1_qk_publication_v3.py:593-650) through ``kf_factored_attention``: against the FP32
oracle, the reference's stored no-RoPE golden vector, the CPU emulation of the reference's
factored kernels, and the standard (unfactored) path of this library."""
import pytest
import torch

import kernelfuser_b200 as kf
from conftest import load_golden
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run(q, k, v, gq, gk, **kw):
    out = kf.factored_attention(*[x.to(DEV) for x in (q, k, v, gq, gk)], **kw)
    torch.cuda.synchronize()
    kf.check_status()
    return out.cpu()


def check(out, ref, emu, label):
    m, me = orc.metric(out, ref), orc.metric(emu, ref)
    assert orc.within_tolerance(m), (label, m)
    # no worse than the reference's factored kernels (their CPU emulation), up to block-size effects
    assert m["max_abs"] <= 1.5 * me["max_abs"] + 2e-3, (label, m, me)
    assert m["mean_abs"] <= 1.5 * me["mean_abs"] + 1e-4, (label, m, me)


@pytest.mark.parametrize("causal", [False, True])
def test_matches_reference_golden(causal):
    meta, t = load_golden("norope_s33_d128_bf16")
    want = t["out_causal" if causal else "out_full"]
    out = run(t["q"], t["k"], t["v"], t["gq"], t["gk"], causal=causal)
    assert orc.within_tolerance(orc.metric(out, want))


@pytest.mark.parametrize("b,s,hq,hkv,d,dtype,causal", [
    (2, 517, 8, 2, 128, torch.bfloat16, True),    # ragged tail, two heads per CTA
    (1, 2048, 32, 8, 128, torch.bfloat16, True),  # the one-tile-per-CTA kernel (automatic choice at this size)
    (2, 390, 6, 2, 128, torch.float16, False),    # odd group size
    (2, 517, 4, 2, 256, torch.bfloat16, True),    # D = 256: raw Q lives in TMEM
    (1, 200, 3, 1, 256, torch.float16, False),
    (1, 64, 2, 2, 256, torch.bfloat16, True),
])
def test_matches_oracle(b, s, hq, hkv, d, dtype, causal):
    q, k, v, gq, gk, _, _ = kf.make_inputs(b, s, hq, hkv, d, dtype=dtype, seed=71, rope=False)
    ref = orc.oracle_fp32(q, k, v, gq, gk, None, None, causal)
    emu = orc.emulate_factored_attention(q, k, v, gq, gk, causal=causal)
    check(run(q, k, v, gq, gk, causal=causal), ref, emu, (b, s, hq, hkv, d, dtype, causal))


@pytest.mark.parametrize("variant", [2, 5])
def test_both_d128_kernels(variant):
    # the two-tile kernel is the automatic choice only beyond 8192 query tiles: ask for it by number
    q, k, v, gq, gk, _, _ = kf.make_inputs(2, 700, 8, 2, 128, seed=74, rope=False)
    ref = orc.oracle_fp32(q, k, v, gq, gk, None, None, True)
    emu = orc.emulate_factored_attention(q, k, v, gq, gk, causal=True)
    check(run(q, k, v, gq, gk, causal=True, variant=variant), ref, emu, variant)
    with pytest.raises(ValueError):
        run(q, k, v, gq, gk, causal=True, variant=3)


def test_prepared_keys_follow_the_factored_contract():
    # KN = r(((k * inv_k) * gk) * gq), one rounding; device rsqrt may differ from the host's in the last bit
    q, k, v, gq, gk, _, _ = kf.make_inputs(2, 130, 4, 2, 128, seed=72, rope=False)
    kn = torch.empty_like(k, device=DEV)
    kf.factored_attention(*[x.to(DEV) for x in (q, k, v, gq, gk)], causal=True, kn=kn)
    torch.cuda.synchronize()
    kf.check_status()
    kf32 = k.float()
    want = (kf32 * torch.rsqrt(kf32.square().sum(-1, keepdim=True) / 128 + 1e-6) * gk.float() * gq.float())
    got = kn.cpu().float()
    spacing = want.abs().clamp_min(2.0 ** -120).log2().floor().exp2() * 2.0 ** -7   # bf16 ulp at each value
    assert ((got - want).abs() <= 1.01 * spacing).all()
    assert (got == want.to(torch.bfloat16).float()).float().mean() > 0.99


def test_agrees_with_the_standard_path_and_honours_scale_eps_and_views():
    b, s, hq, hkv, d = 2, 300, 8, 4, 128
    q, k, v, gq, gk, _, _ = kf.make_inputs(b, s, hq, hkv, d, seed=73, rope=False)
    ref = orc.oracle_fp32(q, k, v, gq, gk, None, None, True, scale=0.07, eps=1e-5)
    # [B,S,H,D] projections viewed as [B,H,S,D]
    views = [t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2) for t in (q, k, v)]
    out = kf.factored_attention(*views, gq.to(DEV), gk.to(DEV), causal=True, scale=0.07, eps=1e-5)
    std = kf.optimized_attention(*[x.to(DEV) for x in (q, k, v, gq, gk)], causal=True, norm_style="legacy",
                                 scale=0.07, eps=1e-5)
    torch.cuda.synchronize()
    kf.check_status()
    assert orc.within_tolerance(orc.metric(out.cpu(), ref))
    assert orc.within_tolerance(orc.metric(out.cpu(), std.float().cpu()))
