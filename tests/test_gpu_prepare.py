"""GPU parity of the row-prepare kernel (through the C ABI) against the CPU
emulation of the reference's ``_rows`` rounding contract
(src/e1_rope_publication_v1.py:551-582)."""
import pytest
import torch

import kernelfuser_b200 as kf
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def ulp_report(got, want):
    """Fraction of elements that differ, and the largest difference in units
    of the 16-bit type's spacing at the magnitude of the row's largest value.
    (A one-place flip of a rounding decision before the rotation is amplified
    relative to a rotated output that nearly cancels, so the spacing is taken
    at row scale, not at the scale of each output value.)"""
    g, w = got.float().cpu(), want.float().cpu()
    diff = (g - w).abs()
    frac = float((diff > 0).float().mean())
    mant = 8 if got.dtype == torch.bfloat16 else 11
    spacing = w.abs().amax(-1, keepdim=True) * (2.0 ** -(mant - 1))
    return frac, float((diff / spacing).max())


@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (128, torch.float16), (256, torch.bfloat16),
                                     (256, torch.float16)])
@pytest.mark.parametrize("style", ["hf", "legacy"])
@pytest.mark.parametrize("rope", [True, False])
def test_prepare_rows_matches_rounding_contract(d, dtype, style, rope):
    b, h, s = 3, 5, 77  # not multiples of the CTA tile or the unroll factor
    q, k, v, gq, gk, cos, sin = kf.make_inputs(b, s, h, h, d, dtype=dtype, theta=1e4, seed=2803, rope=rope)
    want = orc.emulate_rows(k, gk, cos, sin, hf_norm=(style == "hf"))
    dev = torch.device("cuda")
    got = kf.prepare_rows(k.to(dev), gk.to(dev), None if cos is None else cos.to(dev),
                          None if sin is None else sin.to(dev), norm_style=style)
    torch.cuda.synchronize()
    frac, max_ulp = ulp_report(got, want)
    # rsqrt and the sum order may differ in the last place, which now and then flips one rounding
    # decision.  Observed on B200 over all 32 parametrisations (and on 2x8x1500 rows): at most 8.5e-5
    # of the elements differ, by at most 0.73 spacings here (1.26 on the larger tensors).
    assert frac < 5e-4 and max_ulp <= 1.51, (frac, max_ulp)


def test_prepare_rows_strided_views_and_poison():
    # head-sliced (batch-strided) input and output views; untouched memory keeps its poison
    b, h, s, d = 2, 6, 40, 128
    q, k, v, gq, gk, cos, sin = kf.make_inputs(b, s, h, h, d, seed=7)
    dev = torch.device("cuda")
    kd = k.to(dev)
    out = torch.full((b, h, s, d), float("nan"), dtype=k.dtype, device=dev)
    kf.prepare_rows(kd[:, 2:4], gk.to(dev), cos.to(dev), sin.to(dev), out=out[:, 2:4])
    torch.cuda.synchronize()
    want = orc.emulate_rows(k[:, 2:4], gk, cos, sin)
    frac, max_ulp = ulp_report(out[:, 2:4], want)
    assert frac < 5e-4 and max_ulp <= 1.51
    assert torch.isnan(out[:, :2]).all() and torch.isnan(out[:, 4:]).all()


def test_prepare_rows_is_deterministic():
    q, k, v, gq, gk, cos, sin = kf.make_inputs(2, 300, 4, 4, 128, seed=9)
    dev = torch.device("cuda")
    args = (k.to(dev), gk.to(dev), cos.to(dev), sin.to(dev))
    a = kf.prepare_rows(*args)
    b = kf.prepare_rows(*args)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
